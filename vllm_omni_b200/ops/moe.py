"""K10 — mixture-of-experts forward on the grouped tcgen05 GEMM (csrc/moe.cu, gemm_sm100.cu).

``moe_forward`` = route (softmax, top-k, renorm) -> plan (expert segments padded to the
128-row MMA tile) -> dispatch (gather rows expert-major) -> grouped GEMM w13 -> SwiGLU ->
grouped GEMM w2 -> weighted combine.  With expert parallelism a rank passes its local expert
range; pairs routed to other ranks contribute nothing locally and the caller sums the
partial outputs across ranks.  ``moe_reference`` is the dense per-token restatement (the
semantics of vllm_omni/model_executor/models/qwen3_omni/qwen3_moe.py).
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _native as nv
from . import fused

c_int, c_long = ctypes.c_int, ctypes.c_long


def moe_route_reference(logits, k, renorm=True):
    p = torch.softmax(logits.float(), dim=-1)
    w, ids = torch.topk(p, k, dim=-1)
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    return ids.to(torch.int32), w


def moe_reference(x, router_w, w13, w2, k, renorm=True, e_lo=0, e_hi=None):
    """x [T, D]; router_w [E, D]; w13 [E, 2F, D]; w2 [E, D, F]."""
    E = w13.shape[0]
    e_hi = E if e_hi is None else e_hi
    logits = F.linear(x.float(), router_w.float())
    ids, w = moe_route_reference(logits.to(x.dtype), k, renorm)
    out = torch.zeros_like(x, dtype=torch.float32)
    Fd = w2.shape[2]
    for t in range(x.shape[0]):
        for j in range(k):
            e = int(ids[t, j])
            if not (e_lo <= e < e_hi):
                continue
            h = F.linear(x[t].float(), w13[e].float())
            h = F.silu(h[:Fd]) * h[Fd:]
            out[t] += w[t, j] * F.linear(h.to(x.dtype).float(), w2[e].float())
    return out.to(x.dtype)


def padded_rows() -> bool:
    """``OMNI_MOE_PADDED=1`` keeps the first layout (every expert's rows padded to a multiple of 128);
    the default packs the rows of all experts back to back."""
    import os
    return os.environ.get("OMNI_MOE_PADDED", "0") == "1"


class _MoEBuffers:
    """Scratch of the MoE chain for up to ``cap`` tokens.  Every allocation lands in a local first: an
    out-of-memory error half way must not leave an object whose key says "ready" over short buffers."""

    def __init__(self, cap, k, E, D, Fd, device, dtype, pad):
        n_pairs = cap * k
        rows, tiles = _rows_tiles(cap, k, E, pad)
        i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device=device)
        t = dict(ids=i32(cap, k), row_of_pair=i32(n_pairs), tile_expert=i32(tiles), tile_row0=i32(tiles), tile_rows=i32(tiles),
                 offsets=i32(E + 1), n_rows=i32(1), weights=torch.empty(cap, k, dtype=torch.float32, device=device),
                 xp=torch.zeros(rows, D, dtype=dtype, device=device), h13=torch.empty(rows, 2 * Fd, dtype=dtype, device=device),
                 h=torch.empty(rows, Fd, dtype=dtype, device=device), y=torch.empty(rows, D, dtype=dtype, device=device))
        self.__dict__.update(t)


def _rows_tiles(T, k, E, pad):
    n_pairs = T * k
    if pad:
        rows = ((n_pairs + E * 127) + 127) // 128 * 128
        return rows, rows // 128
    # rows back to back: every (token, choice) pair is one row; an expert starts a new M tile, so at most one
    # partly filled tile per expert that got rows
    return n_pairs, min(E, n_pairs) + (n_pairs + 127) // 128


_pool: dict = {}


class MoEWorkspace:
    """Handle a layer keeps for its MoE scratch.  The buffers themselves are shared by every layer of
    the process (layers run one after the other on a stream) and sized by power-of-two token buckets
    that are never freed: a CUDA graph captured at one batch size keeps pointing at live memory when a
    larger prefill comes along, and a 48-layer model holds one set of scratch, not 48."""

    def __init__(self):
        self.key = None

    def get(self, T, k, E, D, Fd, device, dtype):
        pad = padded_rows()
        cap = max(64, 1 << (max(T, 1) - 1).bit_length())
        key = (cap, k, E, D, Fd, str(device), dtype, pad)
        buf = _pool.get(key)
        if buf is None:
            buf = _pool[key] = _MoEBuffers(cap, k, E, D, Fd, device, dtype, pad)
        self.key, self.padded = (T,) + key, pad
        self.max_rows, self.max_tiles = _rows_tiles(T, k, E, pad)
        n_pairs = T * k
        self.ids, self.weights, self.row_of_pair = buf.ids[:T], buf.weights[:T], buf.row_of_pair[:n_pairs]
        self.tile_expert, self.tile_row0, self.tile_rows = (buf.tile_expert[:self.max_tiles], buf.tile_row0[:self.max_tiles],
                                                            buf.tile_rows[:self.max_tiles])
        self.offsets, self.n_rows = buf.offsets, buf.n_rows
        self.xp, self.h13, self.h, self.y = (buf.xp[:self.max_rows], buf.h13[:self.max_rows], buf.h[:self.max_rows],
                                             buf.y[:self.max_rows])
        return self


def moe_forward(x, router_logits, w13, w2, k, renorm=True, e_lo=0, e_hi=None, ws: MoEWorkspace | None = None,
                residual=None, out=None, scatter=None):
    """x [T, D] bf16, router_logits [T, E] bf16, w13 [E_local, 2F, D], w2 [E_local, D, F] (the
    local experts [e_lo, e_hi) of E = router_logits.shape[1]).

    ``scatter = (rows_per_owner, ptrs)`` (GPU, expert parallel): instead of returning the partial
    sum of the local experts, store token t's partial into ``ptrs[t // rows_per_owner]`` (peer
    memory of the rank that owns that block of rows) at local row ``t % rows_per_owner``; the
    cross-rank sum is finished by ``parallel.tensor_parallel.RowParallelReduce.reduce_from``."""
    T, D = x.shape
    E = router_logits.shape[1]
    e_hi = E if e_hi is None else e_hi
    Fd = w2.shape[2]
    if not x.is_cuda:
        ids, w = moe_route_reference(router_logits, k, renorm)
        y = torch.zeros(T, D, dtype=torch.float32)
        for t in range(T):
            for j in range(k):
                e = int(ids[t, j])
                if e_lo <= e < e_hi:
                    h = F.linear(x[t].float(), w13[e - e_lo].float())
                    h = (F.silu(h[:Fd]) * h[Fd:]).to(x.dtype).float()
                    y[t] += w[t, j] * F.linear(h, w2[e - e_lo].float())
        if residual is not None:
            y += residual.float()
        y = y.to(x.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    ws = (ws or MoEWorkspace()).get(T, k, E, D, Fd, x.device, x.dtype)
    lib, st = nv.lib("moe"), nv.stream_ptr()
    assert router_logits.dtype == torch.bfloat16 and router_logits.stride(1) == 1
    nv.check_rc(lib.omni_moe_route(nv.ptr(router_logits), c_int(router_logits.stride(0)), c_int(T), c_int(E), c_int(k),
                                   c_int(1 if renorm else 0), nv.ptr(ws.ids), nv.ptr(ws.weights), st), "omni_moe_route")
    g = nv.lib("gemm_sm100")
    status = nv.status_word(x.device)
    El = w13.shape[0]
    if nv.bounds_check_enabled():
        # checked build: expert ids outside [0, E) and rows outside the expert-major buffers are reported, not used
        lib.omni_moe_set_bounds(c_long(ws.xp.shape[0]), nv.ptr(status))
    if ws.padded:
        nv.check_rc(lib.omni_moe_plan(nv.ptr(ws.ids), c_int(T * k), c_int(E), c_int(e_lo), c_int(e_hi),
                                      c_int(ws.max_tiles), nv.ptr(ws.row_of_pair), nv.ptr(ws.tile_expert),
                                      nv.ptr(ws.offsets), nv.ptr(ws.n_rows), st), "omni_moe_plan")
    else:
        nv.check_rc(lib.omni_moe_plan_compact(nv.ptr(ws.ids), c_int(T * k), c_int(E), c_int(e_lo), c_int(e_hi),
                                              c_int(ws.max_tiles), nv.ptr(ws.row_of_pair), nv.ptr(ws.tile_expert),
                                              nv.ptr(ws.tile_row0), nv.ptr(ws.tile_rows), nv.ptr(ws.n_rows), st),
                    "omni_moe_plan_compact")
    nv.check_rc(lib.omni_moe_dispatch(nv.ptr(x), c_long(x.stride(0)), nv.ptr(ws.row_of_pair), c_int(T * k), c_int(k),
                                      c_int(D), nv.ptr(ws.xp), st), "omni_moe_dispatch")
    # tile_expert holds GLOBAL expert ids; the local weight tensors start at e_lo
    te = ws.tile_expert
    if e_lo:
        te = torch.where(te >= 0, te - e_lo, te)

    def grouped(a, lda, w, c, ldc, n, kk):
        if ws.padded:
            nv.check_rc(g.omni_gemm_bf16_grouped(nv.ptr(a), c_int(lda), nv.ptr(w), c_int(El), nv.ptr(c), c_int(ldc),
                                                 c_int(ws.max_rows), c_int(n), c_int(kk), nv.ptr(te), c_int(0), c_int(0),
                                                 nv.ptr(status), st), "omni_gemm_bf16_grouped")
        else:
            nv.check_rc(g.omni_gemm_bf16_grouped_compact(nv.ptr(a), c_int(lda), nv.ptr(w), c_int(El), nv.ptr(c), c_int(ldc),
                                                         c_int(ws.max_rows), c_int(n), c_int(kk), nv.ptr(te),
                                                         nv.ptr(ws.tile_row0), nv.ptr(ws.tile_rows), c_int(ws.max_tiles),
                                                         c_int(0), c_int(0), nv.ptr(status), st),
                        "omni_gemm_bf16_grouped_compact")
    grouped(ws.xp, D, w13, ws.h13, 2 * Fd, 2 * Fd, D)
    fused.silu_mul(ws.h13, out=ws.h)
    grouped(ws.h, Fd, w2, ws.y, D, D, Fd)
    if scatter is not None:
        per, ptrs = scatter
        arr = (ctypes.c_void_p * len(ptrs))(*ptrs)
        nv.check_rc(lib.omni_moe_combine_scatter(nv.ptr(ws.y), nv.ptr(ws.row_of_pair), nv.ptr(ws.weights), c_int(T), c_int(k),
                                                 c_int(D), c_int(per), arr, st), "omni_moe_combine_scatter")
        return None
    if out is None:
        out = torch.empty_like(x)
    nv.check_rc(lib.omni_moe_combine(nv.ptr(ws.y), nv.ptr(ws.row_of_pair), nv.ptr(ws.weights), c_int(T), c_int(k),
                                     c_int(D), nv.ptr(residual), c_long(residual.stride(0) if residual is not None else 0),
                                     nv.ptr(out), c_long(out.stride(0)), st), "omni_moe_combine")
    return out
