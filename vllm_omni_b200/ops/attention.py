"""K4 — flash attention forward on tcgen05/TMEM (csrc/attention_sm100.cu).

``attention`` takes q/k/v as [B, S, H, D] views with a contiguous head dimension and free
batch / row / head strides, so a packed ``[B, S, 3, H, D]`` projection output is consumed in
place.  The reference reaches PyTorch SDPA on this hardware
(vllm_omni/diffusion/attention/backends/sdpa.py:82); ``attention_reference`` restates that
in fp32 and is the oracle of the numerics tests.
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import _native as nv

c_int, c_long, c_float = ctypes.c_int, ctypes.c_long, ctypes.c_float


class _AttnPrev(ctypes.Structure):
    """Continuation operands of ``omni_attn_fwd_cont`` (csrc/attention_sm100.cu ``AttnPrev``)."""
    _fields_ = [("o", ctypes.c_void_p), ("lse", ctypes.c_void_p), ("rs", ctypes.c_long), ("hs", ctypes.c_long),
                ("bs", ctypes.c_long)]


def attention_reference(q, k, v, scale=None, kv_lens=None, return_lse=False, causal=False, q_offset=0):
    """fp32 softmax(q k^T * scale) v.  q: [B,Sq,H,D], k/v: [B,Skv,Hkv,D]."""
    B, Sq, H, D = q.shape
    Hkv = k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(H // Hkv, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(H // Hkv, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if kv_lens is not None:
        idx = torch.arange(k.shape[1], device=q.device)[None, None, None, :]
        s = s.masked_fill(idx >= kv_lens.to(q.device)[:, None, None, None], float("-inf"))
    if causal:
        qi = torch.arange(Sq, device=q.device)[:, None] + q_offset
        ki = torch.arange(k.shape[1], device=q.device)[None, :]
        s = s.masked_fill((ki > qi)[None, None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    o = torch.matmul(torch.softmax(s, dim=-1), vf).permute(0, 2, 1, 3)
    o = o.to(q.dtype)
    return (o, lse) if return_lse else o


def merge_partials(o_a, lse_a, o_b, lse_b):
    """Combine two attentions of the same queries over disjoint key sets (fp32 restatement of the
    kernel's continuation epilogue): o [B,S,H,D], lse [B,H,S]; rows without any key carry -inf."""
    la, lb = lse_a.transpose(1, 2).unsqueeze(-1), lse_b.transpose(1, 2).unsqueeze(-1)       # [B,S,H,1]
    wb = torch.sigmoid(lb - la)
    wb = torch.where(torch.isinf(lb) & (lb < 0), torch.zeros_like(wb), wb)
    wb = torch.where(torch.isinf(la) & (la < 0) & ~(torch.isinf(lb) & (lb < 0)), torch.ones_like(wb), wb)
    o = o_a.float() * (1 - wb) + o_b.float() * wb
    return o, torch.logaddexp(lse_a, lse_b)


def attention(q, k, v, scale=None, kv_lens=None, out=None, out2=None, split=0, return_lse=False,
              scatter=None, causal=False, q_offset=0, sync=None, merge_prev=None):
    """Non-causal attention.  Returns ``out`` ([B, Sq, H, D], or the given buffer).

    ``out2``/``split``: rows >= split of every batch go to ``out2`` (row index s - split).

    ``scatter = dict(n_peers, rows_per_rank, rows_per_rank2, o_ptrs, o2_ptrs, o_strides, o2_strides)``:
    fused reverse all-to-all; row s < split is stored on rank s // rows_per_rank through the device
    pointer ``o_ptrs[rank]`` (strides = (row, head, batch) in elements), rows >= split likewise with
    the ``*2`` entries.  ``out`` / ``out2`` are then unused.

    ``sync``: an ``OmniSync`` (parallel/peer_memory.py) whose signalling half tells the group that
    this launch's peer stores are out, so the consumer kernel waits for them itself.

    ``merge_prev = (o_prev [B, Sq, H, D], lse_prev [B, H, Sq] fp32)``: the result of the same queries
    over OTHER keys (another sequence-parallel K/V shard); this launch's epilogue stores the
    combination of both, and the combined LSE when ``return_lse``.  ``o_prev`` may be ``out``.
    """
    B, Sq, H, D = q.shape
    Skv, Hkv = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if not q.is_cuda:
        r = attention_reference(q, k, v, scale, kv_lens, return_lse or merge_prev is not None, causal, q_offset)
        o, lse = (r if (return_lse or merge_prev is not None) else (r, None))
        if merge_prev is not None:
            o, lse = merge_partials(merge_prev[0], merge_prev[1], o, lse)
            o = o.to(q.dtype)
        if out2 is not None:
            out.copy_(o[:, :split])
            out2.copy_(o[:, split:])
        elif out is not None:
            out.copy_(o)
        else:
            out = o
        return (out, lse) if return_lse else out
    assert q.dtype == torch.bfloat16 and D in (64, 128), "tcgen05 attention path: bf16, head_dim 64 or 128"
    for t in (q, k, v):
        assert t.stride(3) == 1
    sc = scatter
    if sc is not None:
        os_, o2s = sc["o_strides"], sc.get("o2_strides") or (0, 0, 0)
        op = (ctypes.c_void_p * sc["n_peers"])(*sc["o_ptrs"])
        o2p = (ctypes.c_void_p * sc["n_peers"])(*sc["o2_ptrs"]) if sc.get("o2_ptrs") else None
        out_ptr, out2_ptr = ctypes.c_void_p(sc["o_ptrs"][0]), ctypes.c_void_p(sc["o2_ptrs"][0] if o2p else 0)
        split = sc.get("split", split)
    else:
        if out is None:
            out = torch.empty(B, Sq, H, D, dtype=q.dtype, device=q.device)
        assert out.stride(3) == 1 and (out2 is None or out2.stride(3) == 1)
        os_ = (out.stride(1), out.stride(2), out.stride(0))
        o2s = (out2.stride(1), out2.stride(2), out2.stride(0)) if out2 is not None else (0, 0, 0)
        op = o2p = None
        out_ptr, out2_ptr = nv.ptr(out), nv.ptr(out2)
    lse = torch.empty(B, H, Sq, dtype=torch.float32, device=q.device) if return_lse else None
    if kv_lens is not None:
        assert kv_lens.dtype == torch.int32 and kv_lens.is_cuda
    prev = None
    if merge_prev is not None:
        po, pl = merge_prev
        assert po.dtype == q.dtype and po.shape == (B, Sq, H, D) and po.stride(3) == 1
        assert pl.dtype == torch.float32 and pl.shape == (B, H, Sq) and pl.is_contiguous()
        prev = _AttnPrev(po.data_ptr(), pl.data_ptr(), po.stride(1), po.stride(2), po.stride(0))
    st = nv.status_word(q.device)
    rc = nv.lib("attention_sm100").omni_attn_fwd_cont(
        nv.ptr(q), c_long(q.stride(1)), c_long(q.stride(2)), c_long(q.stride(0)),
        nv.ptr(k), c_long(k.stride(1)), c_long(k.stride(2)), c_long(k.stride(0)),
        nv.ptr(v), c_long(v.stride(1)), c_long(v.stride(2)), c_long(v.stride(0)),
        out_ptr, c_long(os_[0]), c_long(os_[1]), c_long(os_[2]),
        out2_ptr, c_long(o2s[0]), c_long(o2s[1]), c_long(o2s[2]), c_int(split),
        nv.ptr(lse), c_int(B), c_int(H), c_int(Hkv), c_int(Sq), c_int(Skv), c_int(D), nv.ptr(kv_lens),
        c_float(scale), c_int(1 if causal else 0), c_int(q_offset), c_int(sc["n_peers"] if sc else 0), c_int(sc["rows_per_rank"] if sc else 0),
        c_int(sc.get("rows_per_rank2", 0) if sc else 0), op, o2p,
        ctypes.byref(prev) if prev is not None else None,
        ctypes.byref(sync) if sync is not None else None, nv.ptr(st), nv.stream_ptr())
    nv.check_rc(rc, "omni_attn_fwd")
    return (out, lse) if return_lse else out
