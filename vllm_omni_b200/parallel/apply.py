"""Attach the configured parallel strategies to a freshly built pipeline
(the role of the ``_sp_plan`` hook installation in vllm_omni/diffusion/registry.py:122-192)."""
from __future__ import annotations

import os

from . import parallel_state as ps


def apply_parallelism(pipe, od_config) -> None:
    pc = od_config.parallel_config
    tr = getattr(pipe, "transformer", None)
    if tr is not None and getattr(tr, "sp_style", "joint") == "attention" and pc.ulysses_degree * pc.ring_degree > 1:
        # single-stream models shard rows themselves and only need a sequence-parallel attention
        from .sp_attention import SequenceParallelAttention
        for t in (tr, getattr(pipe, "transformer_2", None)):
            if t is not None:
                t.sp = SequenceParallelAttention(ps.get_sp_group(), t.cfg.num_attention_heads, t.cfg.attention_head_dim,
                                                 mode=os.environ.get("OMNI_SP_MODE"))
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
        from .tensor_parallel import shard_transformer
        shard_transformer(tr, ps.get_tp_group())
