"""Attach the configured parallel strategies to a freshly built pipeline
(the role of the ``_sp_plan`` hook installation in vllm_omni/diffusion/registry.py:122-192)."""
from __future__ import annotations

import os

from . import parallel_state as ps


def install_sp_plan(tr, group) -> None:
    """Validate a transformer's declarative ``_sp_plan`` and, for models that ask for it
    (``sp_hooks = True``: custom pipelines and models that do not shard rows in their own forward),
    install the split / gather hooks (vllm_omni/diffusion/hooks/sequence_parallel.py:149,412).  The
    built-in families shard inside ``forward`` / the pipeline loop, where the split costs no extra
    copy and the fused exchange kernels see this rank's rows directly; their plan documents the
    layout and is checked here so that a malformed declaration fails at load, not at run time."""
    from .sp_plan import apply_sp_plan, validate_sp_plan
    plan = getattr(tr, "_sp_plan", None)
    if not plan:
        return
    validate_sp_plan(plan)
    if getattr(tr, "sp_hooks", False) and getattr(tr, "_sp_hook_registry", None) is None:
        tr._sp_hook_registry = apply_sp_plan(tr, plan, group)


def _heads_of(cfg) -> tuple[int, int]:
    """(attention heads, head width) of a transformer config, whichever of the two naming schemes it uses."""
    h = getattr(cfg, "num_attention_heads", None) or getattr(cfg, "n_heads")
    d = getattr(cfg, "attention_head_dim", None) or getattr(cfg, "head_dim")
    return int(h), int(d)


def apply_parallelism(pipe, od_config) -> None:
    pc = od_config.parallel_config
    tr = getattr(pipe, "transformer", None)
    if tr is not None and pc.ulysses_degree * pc.ring_degree > 1:
        for t in (tr, getattr(pipe, "transformer_2", None)):
            if t is not None:
                install_sp_plan(t, ps.get_sp_group())
    if tr is not None and getattr(tr, "sp_style", "joint") == "attention" and pc.ulysses_degree * pc.ring_degree > 1:
        # single-stream models shard rows themselves and only need a sequence-parallel attention
        from .sp_attention import SequenceParallelAttention
        for t in (tr, getattr(pipe, "transformer_2", None)):
            if t is not None:
                t.sp = SequenceParallelAttention(ps.get_sp_group(), *_heads_of(t.cfg), mode=os.environ.get("OMNI_SP_MODE"))
    elif pc.ulysses_degree > 1 and pc.ring_degree > 1 and tr is not None:
        from .hybrid import HybridJointAttention
        tr.sp = HybridJointAttention(ps.get_sp_group(), tr.cfg.num_attention_heads, tr.cfg.attention_head_dim,
                                     mode=os.environ.get("OMNI_SP_MODE"))
    elif pc.ulysses_degree > 1 and tr is not None:
        from .ulysses import UlyssesJointAttention
        mode = os.environ.get("OMNI_SP_MODE")            # "fused" (default on GPU) or "nccl" (baseline)
        tr.sp = UlyssesJointAttention(ps.get_sp_group().ulysses, tr.cfg.num_attention_heads,
                                      tr.cfg.attention_head_dim, mode=mode)
    elif pc.ring_degree > 1 and tr is not None:
        from .ring import RingJointAttention
        tr.sp = RingJointAttention(ps.get_sp_group().ring, tr.cfg.num_attention_heads, tr.cfg.attention_head_dim)
    if pc.cfg_parallel_size > 1:
        from .cfg_parallel import CFGExchange
        pipe.cfg_exchange = CFGExchange(ps.get_cfg_group())
    if pc.tensor_parallel_size > 1 and tr is not None:
        if hasattr(tr, "enable_tensor_parallel"):        # decoder-style denoisers shard themselves (heads + experts)
            tr.enable_tensor_parallel(ps.get_tp_group())
        else:
            from .tensor_parallel import shard_transformer
            shard_transformer(tr, ps.get_tp_group())
