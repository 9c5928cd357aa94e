"""Paged-KV ops: cache write and page gather (csrc/kv_cache.cu) and attention over the paged
cache.  Attention runs on the tcgen05 kernel (csrc/attention_sm100.cu) whose TMA producer walks
the block table: decode maps the query heads that share a KV head onto the rows of one MMA
tile, chunked prefill is the causal kernel with a query offset.  A CUDA-core decode kernel
(csrc/kv_cache.cu) remains for page sizes the TMA path does not take.  CPU paths restate the
same semantics in PyTorch for the engine's CPU tests."""
from __future__ import annotations

import ctypes
import math

import torch

from . import _native as nv

c_int, c_long, c_float = ctypes.c_int, ctypes.c_long, ctypes.c_float


def _set_bounds(k_cache) -> None:
    """Checked build only: tell the library how many slots / pages the cache holds."""
    if nv.bounds_check_enabled():
        nb, bs = k_cache.shape[0], k_cache.shape[1]
        nv.lib("kv_cache").omni_kv_set_bounds(c_long(nb * bs), c_int(nb), nv.ptr(nv.status_word(k_cache.device)))


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
    _set_bounds(k_cache)
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
    _set_bounds(k_cache)
    rc = nv.lib("kv_cache").omni_kv_gather(nv.ptr(k_cache), nv.ptr(v_cache), nv.ptr(block_table), c_int(bs), c_int(T),
                                           c_int(Hkv * D), nv.ptr(out_k), nv.ptr(out_v), nv.stream_ptr())
    nv.check_rc(rc, "omni_kv_gather")
    return out_k, out_v


_scratch: dict = {}


def _scratch_for(device, n_part: int, D: int):
    key = (device.index, n_part)
    sc = _scratch.get(key)
    if sc is None:
        sc = (torch.empty(n_part * D, dtype=torch.float32, device=device),
              torch.empty(n_part * 2, dtype=torch.float32, device=device))
        _scratch[key] = sc
    return sc


def tma_pages_ok(block_size: int, D: int) -> bool:
    """Page shapes the tensor-core path takes: head_dim 128, pages of 8..128 tokens that tile 128."""
    return D == 128 and block_size >= 8 and block_size % 8 == 0 and 128 % block_size == 0


def _attn_paged(q, q_rs, q_hs, q_bs, k_cache, v_cache, block_tables, kv_lens, out, o_rs, o_hs, o_bs, B, H, Hkv, Sq,
                max_kv, scale, causal, q_offset, kv_splits, lse=None):
    nb, bs = k_cache.shape[0], k_cache.shape[1]
    part_o = part_ml = None
    if kv_splits > 1:
        part_o, part_ml = _scratch_for(q.device, B * H * Sq * kv_splits, 128)
    st = nv.status_word(q.device)
    rc = nv.lib("attention_sm100").omni_attn_fwd_paged(
        nv.ptr(q), c_long(q_rs), c_long(q_hs), c_long(q_bs), nv.ptr(k_cache), nv.ptr(v_cache), c_int(nb), c_int(bs),
        nv.ptr(block_tables), c_int(block_tables.stride(0)), nv.ptr(out), c_long(o_rs), c_long(o_hs), c_long(o_bs),
        nv.ptr(lse), c_int(B), c_int(H), c_int(Hkv), c_int(Sq), c_int(max_kv), nv.ptr(kv_lens), c_float(scale),
        c_int(1 if causal else 0), c_int(q_offset), c_int(kv_splits), nv.ptr(part_o), nv.ptr(part_ml), nv.ptr(st),
        nv.stream_ptr())
    nv.check_rc(rc, "omni_attn_fwd_paged")


def paged_decode(q, k_cache, v_cache, block_tables, seq_lens, scale=None, num_splits=None, out=None, impl=None):
    """q: [num_seqs, H, D] (one new token per sequence) -> [num_seqs, H, D].

    ``impl``: "tc" (tcgen05 kernel; default whenever the page shape allows) or "simt"."""
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
    assert q.stride(-1) == 1 and q.stride(1) == D and block_tables.dtype == torch.int32 and seq_lens.dtype == torch.int32
    G = H // Hkv
    if impl is None:
        impl = "tc" if tma_pages_ok(bs, D) and G <= 128 else "simt"
    if impl == "tc":
        # the G heads of a group are the rows of the query tile: row pitch = one head (D),
        # "head" pitch = one group (G * D), batch pitch = one token
        max_kv = block_tables.shape[1] * bs
        tiles = (max_kv + 127) // 128
        if num_splits is None:
            # one CTA per SM: pick the split count with the fewest (fractional) waves of 148 CTAs
            ctas = n * Hkv
            num_splits = min(range(1, min(tiles, 16) + 1),
                             key=lambda sp: -(-ctas * sp // 148) / sp + 0.02 * sp)
        assert out.stride(-1) == 1 and out.stride(1) == D
        _attn_paged(q, D, G * D, q.stride(0), k_cache, v_cache, block_tables, seq_lens, out, D, G * D, out.stride(0),
                    n, Hkv, Hkv, G, max_kv, scale, False, 0, num_splits)
        return out
    if num_splits is None:
        # enough CTAs to fill the GPU: seqs x kv heads x splits >= ~2 waves of 148 SMs
        num_splits = max(1, min(32, (148 * 8 + n * Hkv - 1) // (n * Hkv)))
    sc = _scratch_for(q.device, n * H * num_splits, D)
    rc = nv.lib("kv_cache").omni_paged_decode(
        nv.ptr(q), c_long(q.stride(0)), nv.ptr(k_cache), nv.ptr(v_cache), nv.ptr(block_tables),
        c_int(block_tables.shape[1]), nv.ptr(seq_lens), c_int(n), c_int(bs), c_int(H), c_int(Hkv), c_int(D),
        c_float(scale), c_int(num_splits), nv.ptr(sc[0]), nv.ptr(sc[1]), nv.ptr(out), c_long(out.stride(0)),
        nv.stream_ptr())
    nv.check_rc(rc, "omni_paged_decode")
    return out


def paged_prefill(q, k_cache, v_cache, block_table, kv_len: int, scale=None, out=None):
    """Causal attention of the LAST ``T`` tokens of one sequence against its whole paged context.

    q: [T, H, D]; block_table: int32 [max_blocks]; kv_len: tokens in the cache including these T
    (their K/V already written).  Query row i sees keys [0, kv_len - T + i]."""
    T, H, D = q.shape
    nb, bs, Hkv, _ = k_cache.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty_like(q)
    if not q.is_cuda or not tma_pages_ok(bs, D):
        from .attention import attention, attention_reference
        gk, gv = kv_gather(k_cache, v_cache, block_table, kv_len)
        if q.is_cuda:
            attention(q[None], gk[None], gv[None], scale=scale, causal=True, q_offset=kv_len - T, out=out[None])
        else:
            out.copy_(attention_reference(q[None], gk[None], gv[None], scale, causal=True, q_offset=kv_len - T)[0])
        return out
    assert q.stride(-1) == 1 and out.stride(-1) == 1 and block_table.dtype == torch.int32
    lens = torch.full((1,), kv_len, dtype=torch.int32, device=q.device)
    bt = block_table.view(1, -1)
    _attn_paged(q, q.stride(0), q.stride(1), T * q.stride(0), k_cache, v_cache, bt, lens, out, out.stride(0),
                out.stride(1), T * out.stride(0), 1, H, Hkv, T, kv_len, scale, True, kv_len - T, 1)
    return out
