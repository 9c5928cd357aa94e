"""Tensor parallelism for the DiT blocks (K2).

Column-parallel first GEMM (QKV by head group, MLP up by column block), row-parallel second
GEMM (attention out, MLP down) whose partial sums must be added across ranks.  The reference
uses vLLM's ``ColumnParallelLinear`` / ``RowParallelLinear`` with an NCCL all-reduce after every
row-parallel layer (vllm_omni/diffusion/distributed/parallel_state.py:769).

Here the reduction is folded into the GEMM's output stage: every rank writes its partial tile
into ITS slot of a symmetric peer buffer; after one bounded-wait barrier each rank reduces the
rows it owns by reading all slots over NVLink (reduce-scatter), applies gate/residual on those
rows, and broadcasts them with peer stores (all-gather) — two kernels and two barriers instead
of GEMM + all-reduce + elementwise.  ``mode="nccl"`` keeps the all-reduce baseline (and is the
CPU path).
"""
from __future__ import annotations

import torch

from ..diffusion.layers.linear import FusedLinear


def shard_rows(w: torch.Tensor, rank: int, world: int, groups: int = 1) -> torch.Tensor:
    """Column-parallel shard of an [out, in] weight.  ``groups`` > 1 keeps fused projections
    aligned (e.g. 3 for q|k|v: every rank gets its slice of each of the 3 parts)."""
    out = w.shape[0]
    per = out // groups
    assert per % world == 0, f"{per} rows per group are not divisible by TP size {world}"
    sl = per // world
    parts = [w[g * per + rank * sl: g * per + (rank + 1) * sl] for g in range(groups)]
    return torch.cat(parts, dim=0).contiguous()


def shard_cols(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Row-parallel shard of an [out, in] weight (splits the input features)."""
    k = w.shape[1]
    assert k % world == 0
    sl = k // world
    return w[:, rank * sl:(rank + 1) * sl].contiguous()


class RowParallelReduce:
    """Sum of per-rank partial outputs, then gate * y + residual, identical on every rank."""

    def __init__(self, group, mode: str | None = None):
        self.group = group
        self.P, self.rank = group.world_size, group.rank_in_group
        self.mode = mode or ("peer" if torch.cuda.is_available() else "nccl")
        self.arena = None
        self._key = None

    def _setup(self, y):
        key = (tuple(y.shape), y.dtype, str(y.device))
        if self._key == key:
            return
        self._key = key
        from .peer_memory import PeerArena
        if self.arena is not None:
            self.arena.close()
        nbytes = y.numel() * y.element_size()
        self.arena = PeerArena(self.group, nbytes * (self.P + 1) + 16384, y.device)
        self.slots = self.arena.alloc((self.P,) + tuple(y.shape), y.dtype)     # slot r written by rank r
        self.result = self.arena.alloc(tuple(y.shape), y.dtype)

    def __call__(self, partial: torch.Tensor, bias=None, gate=None, residual=None, out=None):
        if self.P == 1 or self.mode == "nccl" or not partial.is_cuda:
            y = partial.float()
            if self.P > 1:
                y = y.contiguous()
                self.group.all_reduce(y)
            return _finish(y, bias, gate, residual, out, partial.dtype)
        from .peer_memory import tensor_from_ptr
        self._setup(partial)
        P, r = self.P, self.rank
        self.slots.local[r].copy_(partial)
        self.arena.barrier()
        rows = partial.shape[-2]
        per = (rows + P - 1) // P
        lo, hi = min(rows, r * per), min(rows, (r + 1) * per)
        if hi > lo:
            acc = None
            for src in range(P):       # reduce-scatter: pull my rows of every rank's partial over NVLink
                peer = tensor_from_ptr(self.slots.ptrs[src], (P,) + tuple(partial.shape), partial.dtype, partial.device)
                part = peer[src][..., lo:hi, :].float()
                acc = part if acc is None else acc + part
            mine = _finish(acc, bias, _rows(gate, partial, lo, hi), _slice(residual, lo, hi), None, partial.dtype)
            for dst in range(P):       # all-gather: push my finished rows to every rank
                peer = tensor_from_ptr(self.result.ptrs[dst], tuple(partial.shape), partial.dtype, partial.device)
                peer[..., lo:hi, :].copy_(mine)
        self.arena.barrier()
        res = self.result.local
        if out is not None:
            out.copy_(res)
            return out
        return res.clone()

    def close(self):
        if self.arena is not None:
            self.arena.close()
            self.arena = None


def _slice(t, lo, hi):
    return None if t is None else t[..., lo:hi, :]


def _rows(gate, like, lo, hi):
    return gate


def _finish(y, bias, gate, residual, out, dtype):
    if bias is not None:
        y = y + bias.float()
    if gate is not None:
        B = gate.shape[0]
        shp = y.shape
        y = (y.reshape(B, -1, shp[-1]) * gate.float().unsqueeze(1)).reshape(shp)
    if residual is not None:
        y = y + residual.float()
    y = y.to(dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


class TPLinearPair:
    """(column-parallel ``first``, row-parallel ``second``) built from two full ``FusedLinear``s."""

    def __init__(self, first: FusedLinear, second: FusedLinear, group, groups_first: int = 1, reducer=None):
        P, r = group.world_size, group.rank_in_group
        self.first = FusedLinear(first.in_features, first.out_features // P, bias=first.bias is not None,
                                 dtype=first.weight.dtype, device=first.weight.device)
        self.first.weight.data = shard_rows(first.weight.data, r, P, groups_first)
        if first.bias is not None:
            self.first.bias.data = shard_rows(first.bias.data[:, None], r, P, groups_first)[:, 0].contiguous()
        self.second = FusedLinear(second.in_features // P, second.out_features, bias=False, dtype=second.weight.dtype,
                                  device=second.weight.device)
        self.second.weight.data = shard_cols(second.weight.data, r, P)
        self.second_bias = second.bias
        self.reduce = reducer or RowParallelReduce(group)


def shard_transformer(tr, group, mode: str | None = None) -> None:
    """Replace every block's MLP (and, when heads divide, attention projections) of a Qwen-Image
    style transformer by TP pairs.  Heads are split across ranks, so attention itself needs no
    communication."""
    P = group.world_size
    if P == 1:
        return
    H = tr.cfg.num_attention_heads
    if H % P:
        raise ValueError(f"num_attention_heads ({H}) must be divisible by tensor_parallel_size ({P})")
    reducer = RowParallelReduce(group, mode)
    tr.tp_group, tr.tp_reducer = group, reducer
    for blk in tr.blocks:
        for sp in (blk.img, blk.txt):
            sp.tp_attn = TPLinearPair(sp.to_qkv, sp.to_out, group, groups_first=3, reducer=reducer)
            sp.tp_mlp = TPLinearPair(sp.mlp_up, sp.mlp_down, group, reducer=reducer)
            sp.to_qkv = sp.to_out = sp.mlp_up = sp.mlp_down = None
    tr.tp_heads = H // P
