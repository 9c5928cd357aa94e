"""Per-forward context (vllm_omni/diffusion/forward_context.py): engine config, attention
metadata and sequence-parallel bookkeeping that layers read without threading arguments
through every call."""
from __future__ import annotations

from contextlib import contextmanager
from dataclasses import dataclass, field
from typing import Any


@dataclass
class ForwardContext:
    od_config: Any = None
    attn_metadata: Any = None
    split_text_embed_in_sp: bool = False
    sp_padding_size: int = 0
    sp_original_seq_len: int | None = None
    _sp_shard_depth: int = 0
    step_index: int = 0
    num_steps: int = 0
    cfg_branch: str = "cond"           # which CFG branch the transformer call belongs to
    extras: dict = field(default_factory=dict)

    @property
    def sp_active(self) -> bool:
        return self._sp_shard_depth > 0


_ctx: ForwardContext | None = None


def get_forward_context() -> ForwardContext:
    global _ctx
    if _ctx is None:
        _ctx = ForwardContext()
    return _ctx


def is_forward_context_available() -> bool:
    return _ctx is not None


@contextmanager
def set_forward_context(od_config=None, attn_metadata=None, **kw):
    global _ctx
    prev = _ctx
    _ctx = ForwardContext(od_config=od_config, attn_metadata=attn_metadata, **kw)
    try:
        yield _ctx
    finally:
        _ctx = prev
