"""Declarative sequence-parallel plans and the hooks that apply them
(vllm_omni/diffusion/distributed/sp_plan.py, sp_sharding.py, hooks/sequence_parallel.py,
hooks/base.py).

A model declares ``_sp_plan``: which forward arguments are sharded along which dimension
(``SequenceParallelInput``), which module outputs are gathered (``SequenceParallelOutput``) and
which inputs are only partly sharded (``SequenceParallelPartialInput``: a text prefix stays
replicated).  ``apply_sp_plan`` installs pre/post forward hooks that chunk, auto-pad (recording
the pad so that attention can mask it and the gather can strip it) and all-gather.
"""
from __future__ import annotations

from dataclasses import dataclass
from fnmatch import fnmatch
from typing import Any, Callable

import torch
from torch import nn


@dataclass
class SequenceParallelInput:
    split_dim: int
    expected_dims: int | None = None
    split_output: bool = False
    auto_pad: bool = False


@dataclass
class SequenceParallelOutput:
    gather_dim: int
    expected_dims: int | None = None


@dataclass
class SequenceParallelPartialInput:
    split_dim: int
    text_len_source: str              # name of the forward kwarg that holds the replicated prefix length
    expected_dims: int | None = None


def validate_sp_plan(plan: dict) -> None:
    if not isinstance(plan, dict):
        raise TypeError("_sp_plan must be a dict")
    for mod, spec in plan.items():
        if not isinstance(mod, str):
            raise TypeError(f"module key {mod!r} must be a string")
        if isinstance(spec, SequenceParallelOutput):
            continue
        if isinstance(spec, dict):
            for arg, s in spec.items():
                if not isinstance(s, (SequenceParallelInput, SequenceParallelPartialInput, SequenceParallelOutput)):
                    raise TypeError(f"{mod}.{arg}: unsupported plan entry {type(s).__name__}")
                if s.expected_dims is not None and not (-s.expected_dims <= getattr(s, "split_dim", getattr(s, "gather_dim", 0)) < s.expected_dims):
                    raise ValueError(f"{mod}.{arg}: dim out of range for expected_dims={s.expected_dims}")
        else:
            raise TypeError(f"{mod}: plan entry must be a dict of inputs or a SequenceParallelOutput")


def sp_shard(x: torch.Tensor, dim: int, rank: int, world: int, auto_pad: bool = False):
    """Chunk ``x`` along ``dim``; returns (shard, pad) where pad rows were appended to make the
    length divisible."""
    n = x.shape[dim]
    pad = (-n) % world
    if pad:
        if not auto_pad:
            raise ValueError(f"dimension {dim} of size {n} is not divisible by the SP degree {world}")
        shape = list(x.shape)
        shape[dim] = pad
        x = torch.cat([x, x.new_zeros(shape)], dim=dim)
    return x.chunk(world, dim=dim)[rank].contiguous(), pad


def sp_gather(x: torch.Tensor, dim: int, group, pad: int = 0) -> torch.Tensor:
    if group is None or group.world_size == 1:
        return x                       # nothing was gathered, so there is no padding tail to strip
    full = group.all_gather(x, dim=dim)
    if pad:
        idx = [slice(None)] * full.dim()
        idx[dim] = slice(0, full.shape[dim] - pad)
        full = full[tuple(idx)]
    return full


def resolve_modules(root: nn.Module, pattern: str) -> list[tuple[str, nn.Module]]:
    """'' = the root; otherwise names matched with glob wildcards ("blocks.*.attn")."""
    if pattern in ("", "."):
        return [("", root)]
    return [(n, m) for n, m in root.named_modules() if n and fnmatch(n, pattern)]


class HookRegistry:
    """Keeps the handles so the plan can be removed again."""

    def __init__(self):
        self.handles: list = []
        self.state: dict[str, Any] = {"pad": 0, "orig_len": None}

    def remove(self):
        for h in self.handles:
            h.remove()
        self.handles = []


def apply_sp_plan(model: nn.Module, plan: dict, group, rank: int | None = None, world: int | None = None) -> HookRegistry:
    validate_sp_plan(plan)
    rank = group.rank_in_group if rank is None else rank
    world = group.world_size if world is None else world
    reg = HookRegistry()
    for pattern, spec in plan.items():
        for name, mod in resolve_modules(model, pattern):
            if isinstance(spec, SequenceParallelOutput):
                def post(m, args, out, _s=spec):
                    t = out[0] if isinstance(out, tuple) else out
                    g = sp_gather(t, _s.gather_dim, group, reg.state["pad"])
                    return (g,) + tuple(out[1:]) if isinstance(out, tuple) else g
                reg.handles.append(mod.register_forward_hook(post))
                continue

            def pre(m, args, kwargs, _spec=spec):
                kwargs = dict(kwargs)
                for arg, s in _spec.items():
                    if arg not in kwargs or not isinstance(kwargs[arg], torch.Tensor):
                        continue
                    x = kwargs[arg]
                    if s.expected_dims is not None and x.dim() != s.expected_dims:
                        continue
                    if isinstance(s, SequenceParallelPartialInput):
                        tl = int(kwargs.get(s.text_len_source, 0))
                        idx = [slice(None)] * x.dim()
                        idx[s.split_dim] = slice(0, tl)
                        head = x[tuple(idx)]
                        idx[s.split_dim] = slice(tl, None)
                        tail, pad = sp_shard(x[tuple(idx)], s.split_dim, rank, world, True)
                        kwargs[arg] = torch.cat([head, tail], dim=s.split_dim)
                    else:
                        reg.state["orig_len"] = x.shape[s.split_dim]
                        kwargs[arg], pad = sp_shard(x, s.split_dim, rank, world, s.auto_pad)
                        reg.state["pad"] = pad
                return args, kwargs
            reg.handles.append(mod.register_forward_pre_hook(pre, with_kwargs=True))
    return reg
