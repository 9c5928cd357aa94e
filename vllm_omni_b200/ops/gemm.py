"""K1 — linear layers on the tcgen05 GEMM (csrc/gemm_sm100.cu).

``linear`` computes ``epilogue(x @ w.T)`` with the bias, activation, per-batch gate and
residual fused into the GEMM epilogue.  It replaces the cuBLAS path behind the
reference's vLLM ``ColumnParallelLinear`` / ``RowParallelLinear`` / ``QKVParallelLinear``
(vllm_omni/diffusion/models/qwen_image/qwen_image_transformer.py:427-560).
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.nn.functional as F

from . import _native as nv

ACT = {None: 0, "none": 0, "gelu_tanh": 1, "silu": 2}

PAIR_BN = 512   # force_bn value that selects the CTA-pair (cta_group::2, 256 x 256 tile) kernel


def set_pair_mode(auto: bool) -> None:
    """Let the launcher pick the CTA-pair kernel for problems with at least one full wave of
    256 x 256 tiles (``auto=True``) or only when ``force_bn=PAIR_BN`` is passed."""
    nv.lib("gemm_sm100").omni_gemm_set_pair_mode(ctypes.c_int(1 if auto else 0))


def linear_reference(x, w, bias=None, act=None, residual=None, gate=None):
    """Plain PyTorch restatement (fp32 accumulate) used on CPU and as the test oracle.

    ``gate`` has shape [B, N] and ``x`` [B, S, K] (or [M, K] with B dividing M).
    """
    y = F.linear(x.float(), w.float(), None if bias is None else bias.float())
    if act == "gelu_tanh":
        y = F.gelu(y, approximate="tanh")
    elif act == "silu":
        y = F.silu(y)
    if gate is not None:
        B = gate.shape[0]
        shp = y.shape
        y = (y.reshape(B, -1, shp[-1]) * gate.float().unsqueeze(1)).reshape(shp)
    if residual is not None:
        y = y + residual.float()
    return y.to(x.dtype)


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, act: str | None = None,
           residual: torch.Tensor | None = None, gate: torch.Tensor | None = None,
           out: torch.Tensor | None = None, force_bn: int = 0,
           out_rows_per_batch: int = 0, out_batch_stride: int = 0, scatter=None, row_scatter=None,
           sync=None) -> torch.Tensor:
    """y = residual + gate * act(x @ w.T + bias).

    ``out_rows_per_batch`` / ``out_batch_stride`` (elements): row r of the result is stored at
    ``out + (r // rpb) * batch_stride + (r % rpb) * out.stride(-2)``; used to write one stream's
    rows into a joint [B, S_txt + S_img, N] buffer (pass ``out`` as the [B, S_x, N] slice).

    ``scatter = (P, G, ptrs, ld)``: fused all-to-all epilogue.  Column group g (G columns) goes to
    rank g % P, into the buffer at device pointer ``ptrs[g % P]`` (row pitch ``ld`` elements) at
    column (g // P) * G + col % G.  ``out`` is ignored (pass None).

    ``row_scatter = (rows_per_owner, ptrs, ld)``: fused reduce-scatter feed.  Output row r goes to
    rank r // rows_per_owner, as row r % rows_per_owner of the buffer at ``ptrs[that rank]`` (row
    pitch ``ld``).  ``len(ptrs)`` must equal ceil(M / rows_per_owner).  ``out`` is ignored.

    ``sync``: an ``OmniSync`` (parallel/peer_memory.py): arrivals the launch waits for before it reads
    ``x`` (rows that peers write) and / or reports to the group after its own peer stores.

    x: [..., K] bf16 (last dim contiguous), w: [N, K] bf16, bias: [N], residual: [..., N]
    (may be ``out``), gate: [B, N] view (last dim contiguous, any row stride) where the rows
    of x split evenly into B batches.
    """
    if not x.is_cuda:
        y = linear_reference(x, w, bias, act, residual, gate)
        if out is not None:
            out.copy_(y.reshape(out.shape))
            return out
        return y
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "tcgen05 GEMM path is bf16"
    K = x.shape[-1]
    N = w.shape[0]
    x2 = x.reshape(-1, K)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    M = x2.shape[0]
    if w.stride(-1) != 1:
        w = w.contiguous()
    sc_P, sc_G, sc_rows, sc_arr = 0, 0, 0, None
    to_peers = scatter is not None or row_scatter is not None
    if row_scatter is not None:
        sc_rows, ptrs, ldc = row_scatter
        sc_P = len(ptrs)
    elif scatter is not None:
        sc_P, sc_G, ptrs, ldc = scatter
    if to_peers:
        sc_arr = (ctypes.c_void_p * len(ptrs))(*ptrs)
        c_ptr = nv.ptr(x2)                   # placeholder: the kernel writes through the peer pointers only
    else:
        if out is None:
            out = torch.empty(*x.shape[:-1], N, dtype=x.dtype, device=x.device)
        if out_rows_per_batch:
            assert out.stride(-1) == 1
            ldc = out.stride(-2)
        else:
            ldc = out.view(-1, N).stride(0)
        c_ptr = nv.ptr(out)
    res2 = None
    ldr = 0
    if residual is not None:
        res2 = residual.reshape(-1, N)
        assert res2.stride(-1) == 1
        ldr = res2.stride(0)
    gs = 0
    rpb = 0
    if gate is not None:
        assert gate.dim() == 2 and gate.shape[1] == N and gate.stride(1) == 1
        assert M % gate.shape[0] == 0
        rpb = M // gate.shape[0]
        gs = gate.stride(0) if gate.shape[0] > 1 else N
    st = nv.status_word(x.device)
    rc = nv.lib("gemm_sm100").omni_gemm_bf16_sync(
        nv.ptr(x2), ctypes.c_int(x2.stride(0)), nv.ptr(w), ctypes.c_int(w.stride(0)),
        c_ptr, ctypes.c_int(ldc), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
        nv.ptr(bias), nv.ptr(res2), ctypes.c_int(ldr), nv.ptr(gate), ctypes.c_int(gs), ctypes.c_int(rpb),
        ctypes.c_int(ACT[act]), ctypes.c_int(out_rows_per_batch), ctypes.c_long(out_batch_stride),
        ctypes.c_int(sc_P), ctypes.c_int(sc_G), ctypes.c_int(sc_rows), sc_arr, ctypes.c_int(force_bn),
        ctypes.byref(sync) if sync is not None else None, nv.ptr(st), nv.stream_ptr())
    nv.check_rc(rc, "omni_gemm_bf16")
    return None if to_peers else out


class _GemmDesc(ctypes.Structure):
    _fields_ = [("A", ctypes.c_void_p), ("W", ctypes.c_void_p), ("C", ctypes.c_void_p), ("bias", ctypes.c_void_p),
                ("residual", ctypes.c_void_p), ("gate", ctypes.c_void_p), ("c_batch_stride", ctypes.c_long),
                ("lda", ctypes.c_int), ("ldw", ctypes.c_int), ("ldc", ctypes.c_int), ("M", ctypes.c_int),
                ("ldr", ctypes.c_int), ("gate_stride", ctypes.c_int), ("rows_per_batch", ctypes.c_int),
                ("act", ctypes.c_int), ("c_rows_per_batch", ctypes.c_int), ("scatter_P", ctypes.c_int),
                ("scatter_G", ctypes.c_int), ("peer_out", ctypes.c_void_p * 16)]


def _desc(x, w, bias, act, residual, gate, out, out_rows_per_batch, out_batch_stride, keep, scatter=None):
    K, N = x.shape[-1], w.shape[0]
    x2 = x.reshape(-1, K)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    if w.stride(-1) != 1:
        w = w.contiguous()
    M = x2.shape[0]
    d = _GemmDesc()
    if scatter is not None:                  # column groups go to peers; no local output
        P, G, ptrs, ldc = scatter
        d.scatter_P, d.scatter_G = P, G
        for i, pp in enumerate(ptrs):
            d.peer_out[i] = pp
        c_ptr = x2.data_ptr()                # placeholder, never written
    else:
        ldc = out.stride(-2) if out_rows_per_batch else out.view(-1, N).stride(0)
        c_ptr = out.data_ptr()
    d.A, d.W, d.C = x2.data_ptr(), w.data_ptr(), c_ptr
    d.bias = bias.data_ptr() if bias is not None else None
    d.lda, d.ldw, d.ldc, d.M, d.act = x2.stride(0), w.stride(0), ldc, M, ACT[act]
    d.c_rows_per_batch, d.c_batch_stride = out_rows_per_batch, out_batch_stride
    if residual is not None:
        r2 = residual.reshape(-1, N)
        assert r2.stride(-1) == 1
        d.residual, d.ldr = r2.data_ptr(), r2.stride(0)
        keep.append(r2)
    if gate is not None:
        assert gate.dim() == 2 and gate.shape[1] == N and gate.stride(1) == 1 and M % gate.shape[0] == 0
        d.gate, d.rows_per_batch = gate.data_ptr(), M // gate.shape[0]
        d.gate_stride = gate.stride(0) if gate.shape[0] > 1 else N
    keep += [x2, w]
    return d


def linear_pair(a: dict, b: dict, force_pair: bool | None = None, sync=None) -> None:
    """Two linear layers of the same (N, K) in ONE launch (the image and text streams of a
    dual-stream block).  ``a`` / ``b``: keyword sets of ``linear`` — ``x, w, bias, act, residual,
    gate, out`` (``out`` is required unless ``scatter`` is given), optionally ``out_rows_per_batch,
    out_batch_stride, scatter``.  On the
    GPU both problems share the CTA-pair kernel's tile list, so the short one fills the last wave
    of the long one; on CPU they run one after the other.  ``sync`` as in ``linear``: one wait before
    and one report after the pair, whichever way it is launched."""
    xa, xb = a["x"], b["x"]
    if (not xa.is_cuda) or xa.numel() == 0 or xb.numel() == 0:
        for kw in (a, b):
            if kw["x"].numel():
                linear(**kw)
        return
    assert a["w"].shape == b["w"].shape, "the two problems must share N and K"
    keep: list = []
    ds = [_desc(kw["x"], kw["w"], kw.get("bias"), kw.get("act"), kw.get("residual"), kw.get("gate"), kw.get("out"),
                kw.get("out_rows_per_batch", 0), kw.get("out_batch_stride", 0), keep, kw.get("scatter")) for kw in (a, b)]
    N, K = a["w"].shape
    if force_pair is None:                   # tests force the CTA-pair kernel at sizes below one wave
        force_pair = os.environ.get("OMNI_GEMM_DUAL_FORCE") == "1"
    st = nv.status_word(xa.device)
    rc = nv.lib("gemm_sm100").omni_gemm_bf16_dual_sync(ctypes.byref(ds[0]), ctypes.byref(ds[1]), ctypes.c_int(N),
                                                       ctypes.c_int(K), ctypes.c_int(1 if force_pair else 0),
                                                       ctypes.byref(sync) if sync is not None else None, nv.ptr(st),
                                                       nv.stream_ptr())
    nv.check_rc(rc, "omni_gemm_bf16_dual")
