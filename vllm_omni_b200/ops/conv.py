"""K12 — channels-last convolution and the VAE decoder's element-wise kernels.

``conv2d_nhwc`` is an implicit GEMM on the tcgen05 kernel (csrc/gemm_sm100.cu): the A tile of each
(tap, 64-channel block) is one 4-D TMA box of the NHWC input shifted by the tap offset, zero
padding comes from TMA's out-of-bounds fill, bias / SiLU / residual ride in the GEMM epilogue.
The rest (csrc/vae_ops.cu): fused RMS-norm + SiLU per pixel, nearest 2x up-sampling, layout
conversion in and image conversion out.  CPU paths restate the semantics in PyTorch.
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _native as nv
from .gemm import ACT

c_int, c_long = ctypes.c_int, ctypes.c_long


def pack_conv_weight(w: torch.Tensor, bias: torch.Tensor | None, dtype=torch.bfloat16):
    """[Cout, Cin, k, k] -> ([Cout8, k*k * cin_pad] tap-major with zero padding, bias [Cout8]).
    Cout8 = Cout rounded up to 8, cin_pad = Cin rounded up to 64."""
    Cout, Cin, kh, kw = w.shape
    assert kh == kw and kh in (1, 3)
    cin_pad, cout8 = (Cin + 63) // 64 * 64, (Cout + 7) // 8 * 8
    p = torch.zeros(cout8, kh * kw, cin_pad, dtype=dtype, device=w.device)
    p[:Cout, :, :Cin] = w.permute(0, 2, 3, 1).reshape(Cout, kh * kw, Cin).to(dtype)
    b = torch.zeros(cout8, dtype=dtype, device=w.device)
    if bias is not None:
        b[:Cout] = bias.to(dtype)
    return p.reshape(cout8, -1).contiguous(), b


def conv2d_nhwc_reference(x, w_packed, bias, ksize, cin, act=None, residual=None):
    """x [N,H,W,C>=cin]; the packed weight back to [Cout, cin, k, k] and F.conv2d in fp32."""
    cout8 = w_packed.shape[0]
    taps = ksize * ksize
    w = w_packed.view(cout8, taps, -1)[:, :, :cin].float().reshape(cout8, ksize, ksize, cin).permute(0, 3, 1, 2)
    y = F.conv2d(x[..., :cin].float().permute(0, 3, 1, 2), w, bias.float(), padding=ksize // 2).permute(0, 2, 3, 1)
    if act == "silu":
        y = F.silu(y)
    if residual is not None:
        y = y + residual.float()
    return y


def conv2d_nhwc(x, w_packed, bias, ksize: int, cin: int, act=None, residual=None, out=None):
    """x: [N, H, W, ldx] bf16 (ldx >= cin); returns [N, H, W, Cout8]."""
    N, H, W, ldx = x.shape
    cout8 = w_packed.shape[0]
    if not x.is_cuda:
        y = conv2d_nhwc_reference(x, w_packed, bias, ksize, cin, act, residual).to(x.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    assert x.is_contiguous() and x.dtype == torch.bfloat16 and w_packed.dtype == torch.bfloat16
    if out is None:
        out = torch.empty(N, H, W, cout8, dtype=x.dtype, device=x.device)
    st = nv.status_word(x.device)
    rc = nv.lib("gemm_sm100").omni_conv2d_nhwc_bf16(
        nv.ptr(x), c_long(ldx), nv.ptr(w_packed), nv.ptr(out), c_int(out.stride(2)), c_int(N), c_int(H), c_int(W),
        c_int(cin), c_int(cout8), c_int(ksize), nv.ptr(bias), nv.ptr(residual),
        c_int(residual.stride(2) if residual is not None else 0), c_int(ACT[act]), nv.ptr(st), nv.stream_ptr())
    nv.check_rc(rc, "omni_conv2d_nhwc_bf16")
    return out


def rmsnorm_silu_nhwc(x, gamma, silu: bool = True, out=None):
    """Per pixel: x / sqrt(mean_c x^2) * gamma, then SiLU.  x: [..., C]."""
    C = x.shape[-1]
    if not x.is_cuda:
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True).clamp_min(1e-24)) * gamma.float()
        y = (F.silu(y) if silu else y).to(x.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    assert x.is_contiguous()
    if out is None:
        out = torch.empty_like(x)
    rc = nv.lib("vae_ops").omni_rmsnorm_silu_nhwc(nv.ptr(x), c_long(C), nv.ptr(gamma), nv.ptr(out), c_long(C),
                                                  c_long(x.numel() // C), c_int(C), c_int(1 if silu else 0),
                                                  nv.stream_ptr())
    nv.check_rc(rc, "omni_rmsnorm_silu_nhwc")
    return out


def upsample2x_nhwc(x):
    N, H, W, C = x.shape
    if not x.is_cuda:
        return x.repeat_interleave(2, dim=1).repeat_interleave(2, dim=2)
    out = torch.empty(N, 2 * H, 2 * W, C, dtype=x.dtype, device=x.device)
    rc = nv.lib("vae_ops").omni_upsample2x_nhwc(nv.ptr(x), nv.ptr(out), c_int(N), c_int(H), c_int(W), c_int(C),
                                                nv.stream_ptr())
    nv.check_rc(rc, "omni_upsample2x_nhwc")
    return out


def nchw_to_nhwc(x, cpad: int | None = None, dtype=torch.bfloat16):
    N, C, H, W = x.shape
    cpad = cpad or (C + 7) // 8 * 8
    if not x.is_cuda:
        y = torch.zeros(N, H, W, cpad, dtype=dtype)
        y[..., :C] = x.permute(0, 2, 3, 1).to(dtype)
        return y
    x = x.contiguous()
    assert x.dtype in (torch.float32, torch.bfloat16)
    out = torch.empty(N, H, W, cpad, dtype=torch.bfloat16, device=x.device)
    rc = nv.lib("vae_ops").omni_nchw_to_nhwc(nv.ptr(x), c_int(1 if x.dtype == torch.float32 else 0), nv.ptr(out), c_int(N),
                                             c_int(C), c_int(H), c_int(W), c_int(cpad), nv.stream_ptr())
    nv.check_rc(rc, "omni_nchw_to_nhwc")
    return out


def nhwc_to_image(x, uint8: bool = False):
    """x [N,H,W,>=3] -> fp32 [N,3,H,W] clamped to [-1,1], or uint8 [N,H,W,3] in display range."""
    N, H, W, ld = x.shape
    if not x.is_cuda:
        v = x[..., :3].float().clamp(-1, 1)
        return ((v * 0.5 + 0.5) * 255).round().to(torch.uint8) if uint8 else v.permute(0, 3, 1, 2).contiguous()
    out = torch.empty((N, H, W, 3), dtype=torch.uint8, device=x.device) if uint8 else \
        torch.empty((N, 3, H, W), dtype=torch.float32, device=x.device)
    rc = nv.lib("vae_ops").omni_nhwc_to_image(nv.ptr(x), c_long(ld), nv.ptr(out), c_int(N), c_int(H), c_int(W),
                                              c_int(0 if uint8 else 1), nv.stream_ptr())
    nv.check_rc(rc, "omni_nhwc_to_image")
    return out
