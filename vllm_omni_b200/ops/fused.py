"""Python entry points of the bandwidth-bound fused kernels (csrc/elementwise.cu).

Every function has a plain PyTorch fp32 restatement (``*_reference``) that runs on CPU
and is the oracle of the GPU numerics tests.
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _native as nv

c_int, c_long, c_float = ctypes.c_int, ctypes.c_long, ctypes.c_float


# ------------------------------------------------------------------ norm + modulate (K7)
def norm_modulate_reference(x, weight=None, bias=None, shift=None, scale=None, rms=False, eps=1e-6):
    xf = x.float()
    if rms:
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    else:
        y = F.layer_norm(xf, (x.shape[-1],), None, None, eps)
    if weight is not None:
        y = y * weight.float()
    if bias is not None:
        y = y + bias.float()
    if scale is not None:
        y = y * (1.0 + scale.float().unsqueeze(1))
    if shift is not None:
        y = y + shift.float().unsqueeze(1)
    return y.to(x.dtype)


def norm_modulate(x, weight=None, bias=None, shift=None, scale=None, rms=False, eps=1e-6, out=None):
    """y = norm(x) [* weight + bias] * (1 + scale[b]) + shift[b].

    x: [B, S, D] (or [M, D] when no modulation); shift/scale: [B, D] views with unit inner
    stride (row stride free, e.g. chunks of the [B, 6D] AdaLN projection).
    """
    if not x.is_cuda:
        if (shift is not None or scale is not None) and x.dim() == 2:
            B = (shift if shift is not None else scale).shape[0]
            y = norm_modulate_reference(x.view(B, -1, x.shape[-1]), weight, bias, shift, scale, rms, eps).view_as(x)
        else:
            y = norm_modulate_reference(x, weight, bias, shift, scale, rms, eps)
        if out is not None:
            out.copy_(y)
            return out
        return y
    D = x.shape[-1]
    x2 = x.reshape(-1, D)
    assert x2.stride(1) == 1 and x.dtype == torch.bfloat16
    rows = x2.shape[0]
    if out is None:
        out = torch.empty_like(x, memory_format=torch.contiguous_format)
    o2 = out.view(-1, D)
    mod = shift if shift is not None else scale
    mod_stride, rpb = 0, rows
    if mod is not None:
        assert mod.dim() == 2 and mod.stride(1) == 1
        if shift is not None and scale is not None:
            assert shift.stride(0) == scale.stride(0)
        mod_stride = mod.stride(0) if mod.shape[0] > 1 else D
        rpb = rows // mod.shape[0]
    rc = nv.lib("elementwise").omni_norm_modulate(
        nv.ptr(x2), nv.ptr(o2), c_int(rows), c_int(D), c_int(x2.stride(0)), c_int(o2.stride(0)),
        nv.ptr(weight), nv.ptr(bias), nv.ptr(shift), nv.ptr(scale), c_int(mod_stride), c_int(rpb),
        c_int(1 if rms else 0), c_float(eps), nv.stream_ptr())
    nv.check_rc(rc, "omni_norm_modulate")
    return out


# ------------------------------------------------------------------ qk norm + rope (K7 + K8)
def apply_rope_reference(x, cos, sin, interleaved):
    """x: [..., S, H, D]; cos/sin: [S, D/2] (already gathered per position)."""
    xf = x.float()
    c = cos.float()[:, None, :]
    s = sin.float()[:, None, :]
    if interleaved:
        a, b = xf[..., 0::2], xf[..., 1::2]
        out = torch.stack((a * c - b * s, a * s + b * c), dim=-1).flatten(-2)
    else:
        h = x.shape[-1] // 2
        a, b = xf[..., :h], xf[..., h:]
        out = torch.cat((a * c - b * s, b * c + a * s), dim=-1)
    return out


def qk_norm_rope_reference(qkv, H, Hkv, D, wq, wk, wq_alt, wk_alt, s_alt, cos, sin, interleaved, eps, positions=None):
    B, S = qkv.shape[:2]
    flat = qkv.reshape(B, S, -1).float()
    q = flat[..., : H * D].reshape(B, S, H, D)
    k = flat[..., H * D: (H + Hkv) * D].reshape(B, S, Hkv, D)
    v = flat[..., (H + Hkv) * D:]

    def rn(t, w, wt):
        if w is None:
            return t
        n = t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps)
        out = n * w.float()
        if wt is not None and s_alt < t.shape[1]:
            out = torch.cat((out[:, :s_alt], n[:, s_alt:] * wt.float()), dim=1)
        return out

    q, k = rn(q, wq, wq_alt), rn(k, wk, wk_alt)
    if cos is not None:
        if positions is not None:
            outq = torch.stack([apply_rope_reference(q[b], cos[positions[b].long()], sin[positions[b].long()], interleaved) for b in range(B)])
            outk = torch.stack([apply_rope_reference(k[b], cos[positions[b].long()], sin[positions[b].long()], interleaved) for b in range(B)])
            q, k = outq, outk
        else:
            q, k = apply_rope_reference(q, cos[:S], sin[:S], interleaved), apply_rope_reference(k, cos[:S], sin[:S], interleaved)
    out = torch.cat((q.reshape(B, S, -1), k.reshape(B, S, -1), v), dim=-1)
    return out.to(qkv.dtype).view_as(qkv)


def qk_norm_rope_(qkv, H, Hkv, D, wq=None, wk=None, wq_alt=None, wk_alt=None, s_alt=1 << 30, cos=None, sin=None,
                  interleaved=True, eps=1e-6, positions=None, sync=None):
    """In place on a packed qkv buffer [B, S, (H + 2*Hkv) * D]: q,k <- rope(rmsnorm(q,k)).

    Rows s >= s_alt use the norm weights ``wq_alt`` / ``wk_alt`` (the text rows that follow
    the image rows of a joint sequence).  ``sync``: an ``OmniSync`` whose waiting half names the
    arrivals (peers' QKV epilogues) the kernel waits for before it touches the buffer."""
    if not qkv.is_cuda:
        qkv.copy_(qk_norm_rope_reference(qkv, H, Hkv, D, wq, wk, wq_alt, wk_alt, s_alt, cos, sin, interleaved, eps, positions))
        return qkv
    B, S = qkv.shape[:2]
    assert qkv.dtype == torch.bfloat16 and qkv.stride(-1) == 1 and qkv.is_contiguous()
    ld = qkv.stride(1)
    if cos is not None:
        assert cos.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous() and cos.shape[-1] == D // 2
    if positions is not None:
        assert positions.dtype == torch.int32 and positions.is_contiguous()
    rc = nv.lib("elementwise").omni_qk_norm_rope_sync(
        nv.ptr(qkv), c_int(B), c_int(S), c_int(H), c_int(Hkv), c_int(D), c_int(ld), nv.ptr(wq), nv.ptr(wk),
        nv.ptr(wq_alt), nv.ptr(wk_alt), c_int(min(s_alt, 1 << 30)), nv.ptr(cos), nv.ptr(sin), c_int(1 if interleaved else 0),
        c_float(eps), nv.ptr(positions), ctypes.byref(sync) if sync is not None else None,
        nv.ptr(nv.status_word(qkv.device)), nv.stream_ptr())
    nv.check_rc(rc, "omni_qk_norm_rope")
    return qkv


# ------------------------------------------------------------------ CFG mix + Euler (K6, local part)
def cfg_euler_step_reference(pos, neg, lat, guidance, dt, renorm):
    p = pos.float()
    if neg is None:
        v = p
    else:
        n = neg.float()
        v = n + guidance * (p - n)
        if renorm:
            v = v * (p.norm(dim=-1, keepdim=True) / v.norm(dim=-1, keepdim=True).clamp_min(1e-12))
    return lat + dt * v


def cfg_euler_step_(pos, neg, lat, guidance: float, dt: float, renorm: bool = False, lat_lowp=None,
                    pos_ptr: int | None = None, neg_ptr: int | None = None):
    """lat (fp32, in place) += dt * guided velocity; optional bf16 copy in ``lat_lowp``.

    ``pos_ptr`` / ``neg_ptr``: raw device pointers (bf16, same shape as ``lat``) used instead of
    the tensors; a pointer into a peer GPU's memory makes this the fused CFG exchange."""
    if not lat.is_cuda:
        lat.copy_(cfg_euler_step_reference(pos, neg, lat, guidance, dt, renorm))
        if lat_lowp is not None:
            lat_lowp.copy_(lat)
        return lat
    C = lat.shape[-1]
    rows = lat.numel() // C
    assert lat.dtype == torch.float32 and lat.is_contiguous()
    if pos_ptr is None:
        assert pos.is_contiguous() and pos.dtype == torch.bfloat16
        assert neg is None or (neg.is_contiguous() and neg.dtype == torch.bfloat16)
    p_arg = nv.ptr(pos) if pos_ptr is None else ctypes.c_void_p(pos_ptr)
    n_arg = nv.ptr(neg) if neg_ptr is None else ctypes.c_void_p(neg_ptr)
    rc = nv.lib("elementwise").omni_cfg_euler_step(
        p_arg, n_arg, nv.ptr(lat), nv.ptr(lat_lowp), c_long(rows), c_int(C), c_float(guidance),
        c_float(dt), c_int(1 if renorm else 0), nv.stream_ptr())
    nv.check_rc(rc, "omni_cfg_euler_step")
    return lat


# ------------------------------------------------------------------ SwiGLU (K9)
def silu_mul(x, out=None):
    N = x.shape[-1] // 2
    if not x.is_cuda:
        y = (F.silu(x[..., :N].float()) * x[..., N:].float()).to(x.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    x2 = x.reshape(-1, 2 * N)
    assert x2.stride(1) == 1 and x.dtype == torch.bfloat16
    if out is None:
        out = torch.empty(*x.shape[:-1], N, dtype=x.dtype, device=x.device)
    o2 = out.view(-1, N)
    rc = nv.lib("elementwise").omni_silu_mul(nv.ptr(x2), nv.ptr(o2), c_long(x2.shape[0]), c_int(N),
                                             c_int(x2.stride(0)), c_int(o2.stride(0)), nv.stream_ptr())
    nv.check_rc(rc, "omni_silu_mul")
    return out


# ------------------------------------------------------------------ TeaCache metric (K14)
class RelL1State:
    """Device-resident TeaCache accumulator: [accumulated, last_rel_l1, skip, n_skipped].

    The decision never leaves the GPU unless the caller reads ``skip`` (the reference
    synchronises with ``.cpu().item()`` every step, teacache/hook.py:185-232).
    """

    def __init__(self, device, coefficients=None, thresh: float = 0.2):
        self.state = torch.zeros(4, dtype=torch.float32, device=device)
        coefficients = list(coefficients) if coefficients is not None else []
        self.coef = torch.tensor(coefficients, dtype=torch.float32, device=device) if coefficients else None
        self.ncoef = len(coefficients)
        self.thresh = float(thresh)
        self.scratch = None

    def reset(self):
        self.state.zero_()


def rel_l1_reference(a, b):
    return ((a.float() - b.float()).abs().mean() / (b.float().abs().mean() + 1e-8))


def rel_l1_update(a, b, st: RelL1State, force_compute: bool = False):
    """Accumulate the rescaled rel-L1 distance of ``a`` w.r.t. ``b`` into ``st``; afterwards
    ``st.state[2]`` is 1.0 when the transformer blocks may be skipped this step."""
    if not a.is_cuda:
        rel = float(rel_l1_reference(a, b))
        r = rel
        if st.ncoef:
            r = 0.0
            for c in st.coef.tolist():
                r = r * rel + c
        acc = float(st.state[0]) + abs(r)        # |rescale(rel)|, as the reference accumulates it
        skip = 0.0
        if (not force_compute) and acc < st.thresh:
            skip = 1.0
        else:
            acc = 0.0
        st.state[0] = acc
        st.state[1] = rel
        st.state[2] = skip
        st.state[3] += skip
        return st.state
    assert a.is_contiguous() and b.is_contiguous() and a.dtype == torch.bfloat16 and a.numel() == b.numel()
    n = a.numel()
    lib = nv.lib("elementwise")
    parts = lib.omni_rel_l1_parts(c_long(n))
    if st.scratch is None or st.scratch.numel() < 2 * parts:
        st.scratch = torch.empty(2 * parts, dtype=torch.float32, device=a.device)
    rc = lib.omni_rel_l1(nv.ptr(a), nv.ptr(b), c_long(n), nv.ptr(st.scratch), nv.ptr(st.state), nv.ptr(st.coef),
                         c_int(st.ncoef), c_float(st.thresh), c_int(1 if force_compute else 0), nv.ptr(None),
                         nv.stream_ptr())
    nv.check_rc(rc, "omni_rel_l1")
    return st.state
