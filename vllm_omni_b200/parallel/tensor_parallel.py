"""Tensor parallelism for the DiT blocks (K2).

Column-parallel first GEMM (QKV by head group, MLP up by column block), row-parallel second
GEMM (attention out, MLP down) whose partial sums must be added across ranks.  The reference
uses vLLM's ``ColumnParallelLinear`` / ``RowParallelLinear`` with an NCCL all-reduce after every
row-parallel layer (vllm_omni/diffusion/distributed/parallel_state.py:769).

Here the reduce-scatter is folded into the GEMM: its epilogue stores every output tile through
NVLink into the slot this rank owns on the rank that owns those rows (csrc/gemm_sm100.cu,
``scatter_rows``), so the transfer overlaps the main loop tile by tile.  After one bounded-wait
barrier each rank adds the P slots of its rows from LOCAL memory, applies bias / gate / residual
and stores the finished rows to every rank (csrc/tp_reduce.cu), then a second barrier.
``mode="nccl"`` keeps the all-reduce baseline (and is the CPU path).
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
    """Row-parallel linear layer: ``y = residual + gate * (sum_r x_r @ w_r.T + bias)`` where rank r
    holds the r-th slice of the input features, identical on every rank afterwards.

    ``mode="peer"``: the GEMM's epilogue stores each 128-row tile of its partial product straight
    into the slot reserved for this rank on the rank that owns those rows (NVLink stores while
    the main loop runs on the next tile), one bounded barrier, a reduce kernel that reads only
    local memory and stores the finished rows to every rank, one barrier.
    ``mode="nccl"`` is GEMM + all-reduce + eager epilogue (baseline, and the CPU path).
    """

    def __init__(self, group, mode: str | None = None):
        self.group = group
        self.P, self.rank = group.world_size, group.rank_in_group
        self.mode = mode or ("peer" if torch.cuda.is_available() else "nccl")
        self._states: dict = {}      # (M, N, dtype, device) -> (arena, slots, result, rows per owner)

    def _setup(self, M, N, dtype, device):
        key = (M, N, dtype, str(device))
        st = self._states.get(key)
        if st is None:
            from .peer_memory import PeerArena
            P = self.P
            per = (-(-M // P) + 7) // 8 * 8
            esz = torch.empty(0, dtype=dtype).element_size()
            arena = PeerArena(self.group, (P * per * N + M * N) * esz + 65536, device)
            slots = arena.alloc((P, per, N), dtype)      # slot s: rank s's partial of MY rows
            result = arena.alloc((M, N), dtype)
            st = self._states[key] = (arena, slots, result, per)
        self.arena, self.slots, self.result, self.per = st

    def linear(self, layer: FusedLinear, x: torch.Tensor, bias=None, gate=None, residual=None, out=None,
               capacity: int | None = None):
        """``layer`` holds this rank's [N, K/P] weight slice, ``x`` its [.., K/P] input slice.
        ``capacity`` (>= rows of x): size the peer buffers for this many rows, so that callers whose
        row count changes from call to call (AR decode) reuse one arena per capacity bucket."""
        N = layer.out_features
        if self.P == 1 or self.mode == "nccl" or not x.is_cuda:
            partial = layer(x)
            return self(partial, bias=bias, gate=gate, residual=residual, out=out)
        from ..ops import gemm
        x2 = x.reshape(-1, x.shape[-1])
        res = self.reduce_from(lambda per, ptrs: gemm.linear(x2, layer.weight, None, row_scatter=(per, ptrs, N)),
                               x2.shape[0], N, x.dtype, x.device, bias=bias, gate=gate, residual=residual,
                               capacity=capacity)
        res = res.view(*x.shape[:-1], N)
        if out is not None:
            out.copy_(res)
            return out
        return res.clone()

    def reduce_from(self, produce, M: int, N: int, dtype, device, bias=None, gate=None, residual=None,
                    capacity: int | None = None):
        """Sum over the ranks of an [M, N] partial result that ``produce(rows_per_owner, ptrs)``
        writes straight into peer memory: row r goes to ``ptrs[r // rows_per_owner]`` at local row
        ``r % rows_per_owner`` (pitch N).  Returns the [M, N] view of the reduced result (with bias,
        gate and residual applied) that every rank holds after the second barrier; it is valid
        until the next call with the same shape.  ``capacity`` >= M sizes the buffers (and fixes the
        rows-per-owner split) for callers whose M changes from call to call, so that one arena per
        capacity bucket serves them all."""
        import ctypes
        from ..ops import _native as nv
        self._setup(capacity or M, N, dtype, device)
        P, r, per = self.P, self.rank, self.per
        esz = torch.empty(0, dtype=dtype).element_size()
        owners = -(-M // per)
        # my partial of owner o's rows lands in slot r of owner o
        ptrs = [self.slots.ptrs[o] + r * per * N * esz for o in range(owners)]
        produce(per, ptrs)
        self.arena.barrier()
        lo, hi = min(M, r * per), min(M, (r + 1) * per)
        rpb = 0
        gs = 0
        if gate is not None:
            assert gate.dim() == 2 and gate.stride(1) == 1 and M % gate.shape[0] == 0
            rpb = M // gate.shape[0]
            gs = gate.stride(0) if gate.shape[0] > 1 else N
        res2 = residual.reshape(-1, N) if residual is not None else None
        arr = (ctypes.c_void_p * P)(*self.result.ptrs)
        rc = nv.lib("tp_reduce").omni_tp_reduce_gather(
            nv.ptr(self.slots.local), ctypes.c_int(P), ctypes.c_int(per), ctypes.c_int(N), ctypes.c_int(lo),
            ctypes.c_int(hi - lo), nv.ptr(bias), nv.ptr(gate), ctypes.c_int(gs), ctypes.c_int(rpb), nv.ptr(res2),
            ctypes.c_long(res2.stride(0) if res2 is not None else 0), arr, ctypes.c_long(N), nv.stream_ptr())
        nv.check_rc(rc, "omni_tp_reduce_gather")
        self.arena.barrier()
        return self.result.local[:M]

    def __call__(self, partial: torch.Tensor, bias=None, gate=None, residual=None, out=None):
        """All-reduce form: ``partial`` is this rank's full-size partial product."""
        y = partial.float()
        if self.P > 1:
            y = y.contiguous()
            self.group.all_reduce(y)
        return _finish(y, bias, gate, residual, out, partial.dtype)

    def close(self):
        for arena, *_ in self._states.values():
            arena.close()
        self._states.clear()


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

    def up(self, x, **kw):
        """Column-parallel half: this rank's slice of the output features."""
        return self.first(x, **kw)

    def down(self, h, gate=None, residual=None, out=None):
        """Row-parallel half on this rank's slice ``h`` of the input features; full result."""
        return self.reduce.linear(self.second, h, bias=self.second_bias, gate=gate, residual=residual, out=out)


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
    # FLUX-family single-stream blocks: linear1 = [q | k | v | mlp] rows, linear2 = [attn | mlp] input features
    for blk in getattr(tr, "single_blocks", []) or []:
        shard_flux_single_block(blk, tr.cfg.inner_dim, group)


def shard_flux_single_block(blk, D: int, group) -> None:
    """Column-parallel ``linear1`` (this rank's heads of q, k and v and its slice of the MLP columns)
    and row-parallel ``linear2`` (the matching input features; its bias is applied once, by the
    reduce)."""
    P, r = group.world_size, group.rank_in_group
    F_ = blk.linear1.out_features - 3 * D
    if D % P or F_ % P:
        raise ValueError(f"attention width {D} and MLP width {F_} must be divisible by tensor_parallel_size {P}")
    Dl, Fl = D // P, F_ // P
    w1, b1 = blk.linear1.weight.data, (blk.linear1.bias.data if blk.linear1.bias is not None else None)
    rows = torch.cat([torch.arange(g * D + r * Dl, g * D + (r + 1) * Dl) for g in range(3)] +
                     [torch.arange(3 * D + r * Fl, 3 * D + (r + 1) * Fl)]).to(w1.device)
    lin1 = FusedLinear(w1.shape[1], rows.numel(), bias=b1 is not None, dtype=w1.dtype, device=w1.device)
    lin1.weight.data = w1[rows].contiguous()
    if b1 is not None:
        lin1.bias.data = b1[rows].contiguous()
    w2 = blk.linear2.weight.data
    cols = torch.cat([torch.arange(r * Dl, (r + 1) * Dl), torch.arange(D + r * Fl, D + (r + 1) * Fl)]).to(w2.device)
    lin2 = FusedLinear(cols.numel(), w2.shape[0], bias=False, dtype=w2.dtype, device=w2.device)
    lin2.weight.data = w2[:, cols].contiguous()
    blk.linear2_bias = blk.linear2.bias
    blk.linear1, blk.linear2 = lin1, lin2
