"""Paged-KV ops (csrc/kv_cache.cu): cache write, page gather, split-context decode attention.
CPU paths restate the same semantics in PyTorch for the engine's CPU tests."""
from __future__ import annotations

import ctypes
import math

import torch

from . import _native as nv

c_int, c_long, c_float = ctypes.c_int, ctypes.c_long, ctypes.c_float


def kv_write(k, v, k_cache, v_cache, slots):
    """k, v: [T, Hkv, D]; caches: [num_blocks, block_size, Hkv, D]; slots int32 [T] (<0 = skip)."""
    T = k.shape[0]
    row = k_cache.shape[2] * k_cache.shape[3]
    if not k.is_cuda:
        kf, vf = k_cache.view(-1, row), v_cache.view(-1, row)
        ok = slots >= 0
        kf[slots[ok].long()] = k.reshape(T, row)[ok]
        vf[slots[ok].long()] = v.reshape(T, row)[ok]
        return
    assert k.stride(-1) == 1 and k.stride(1) == k.shape[2] and slots.dtype == torch.int32
    rc = nv.lib("kv_cache").omni_kv_write(nv.ptr(k), nv.ptr(v), c_long(k.stride(0)), c_long(v.stride(0)),
                                          nv.ptr(k_cache), nv.ptr(v_cache), nv.ptr(slots), c_int(T), c_int(row),
                                          nv.stream_ptr())
    nv.check_rc(rc, "omni_kv_write")


def kv_gather(k_cache, v_cache, block_table, T, out_k=None, out_v=None):
    """Pages of one sequence -> contiguous [T, Hkv, D] tensors (or the given buffers, which may
    live in another GPU's peer-mapped memory)."""
    nb, bs, Hkv, D = k_cache.shape
    if out_k is None:
        out_k = torch.empty(T, Hkv, D, dtype=k_cache.dtype, device=k_cache.device)
        out_v = torch.empty_like(out_k)
    if not k_cache.is_cuda:
        idx = (block_table[: (T + bs - 1) // bs].long()[:, None] * bs + torch.arange(bs)[None, :]).reshape(-1)[:T]
        out_k.copy_(k_cache.view(-1, Hkv, D)[idx])
        out_v.copy_(v_cache.view(-1, Hkv, D)[idx])
        return out_k, out_v
    rc = nv.lib("kv_cache").omni_kv_gather(nv.ptr(k_cache), nv.ptr(v_cache), nv.ptr(block_table), c_int(bs), c_int(T),
                                           c_int(Hkv * D), nv.ptr(out_k), nv.ptr(out_v), nv.stream_ptr())
    nv.check_rc(rc, "omni_kv_gather")
    return out_k, out_v


_scratch: dict = {}


def paged_decode(q, k_cache, v_cache, block_tables, seq_lens, scale=None, num_splits=None, out=None):
    """q: [num_seqs, H, D] (one new token per sequence) -> [num_seqs, H, D]."""
    n, H, D = q.shape
    nb, bs, Hkv, _ = k_cache.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty_like(q)
    if not q.is_cuda:
        from .attention import attention_reference
        for i in range(n):
            L = int(seq_lens[i])
            gk, gv = kv_gather(k_cache, v_cache, block_tables[i], L)
            out[i] = attention_reference(q[i:i + 1, None].reshape(1, 1, H, D), gk[None], gv[None], scale)[0, 0]
        return out
    if num_splits is None:
        # enough CTAs to fill the GPU: seqs x kv heads x splits >= ~2 waves of 148 SMs
        num_splits = max(1, min(32, (148 * 8 + n * Hkv - 1) // (n * Hkv)))
    key = (q.device.index, n * H * num_splits)
    sc = _scratch.get(key)
    if sc is None:
        sc = (torch.empty(n * H * num_splits * D, dtype=torch.float32, device=q.device),
              torch.empty(n * H * num_splits * 2, dtype=torch.float32, device=q.device))
        _scratch[key] = sc
    assert q.stride(-1) == 1 and q.stride(1) == D and block_tables.dtype == torch.int32 and seq_lens.dtype == torch.int32
    rc = nv.lib("kv_cache").omni_paged_decode(
        nv.ptr(q), c_long(q.stride(0)), nv.ptr(k_cache), nv.ptr(v_cache), nv.ptr(block_tables),
        c_int(block_tables.shape[1]), nv.ptr(seq_lens), c_int(n), c_int(bs), c_int(H), c_int(Hkv), c_int(D),
        c_float(scale), c_int(num_splits), nv.ptr(sc[0]), nv.ptr(sc[1]), nv.ptr(out), c_long(out.stride(0)),
        nv.stream_ptr())
    nv.check_rc(rc, "omni_paged_decode")
    return out
