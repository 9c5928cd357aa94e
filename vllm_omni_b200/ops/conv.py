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


# ------------------------------------------------------------------ K15: vocoder stacks, channels-last [B, T, C]
def pack_conv1d_weight(w: torch.Tensor, bias: torch.Tensor | None, dtype=torch.bfloat16):
    """[Cout, Cin, k] -> ([Cout8, k * cin_pad] tap-major with zero padding, bias [Cout8])."""
    Cout, Cin, k = w.shape
    cin_pad, cout8 = (Cin + 63) // 64 * 64, (Cout + 7) // 8 * 8
    p = torch.zeros(cout8, k, cin_pad, dtype=dtype, device=w.device)
    p[:Cout, :, :Cin] = w.permute(0, 2, 1).to(dtype)
    b = torch.zeros(cout8, dtype=dtype, device=w.device)
    if bias is not None:
        b[:Cout] = bias.to(dtype)
    return p.reshape(cout8, -1).contiguous(), b


def conv1d_nlc_reference(x, w_packed, bias, k, cin, dil=1, pad=0, t_out=None, act=None, residual=None):
    """fp32 restatement: y[b, t] = sum_j x[b, t + j*dil - pad] W_j^T, zeros outside the input."""
    B, T, _ = x.shape
    t_out = T if t_out is None else t_out
    cout8 = w_packed.shape[0]
    w = w_packed.view(cout8, k, -1)[:, :, :cin].float().permute(0, 2, 1)            # [Cout8, cin, k]
    right = max(0, (t_out - 1) + (k - 1) * dil - pad - (T - 1))
    xp = F.pad(x[..., :cin].float().transpose(1, 2), (max(pad, 0), right))
    if pad < 0:
        xp = xp[..., -pad:]
    y = F.conv1d(xp, w, bias.float(), dilation=dil)[..., :t_out].transpose(1, 2)
    if act == "silu":
        y = F.silu(y)
    if residual is not None:
        y = y + residual.float()
    return y


def conv1d_nlc(x, w_packed, bias, k: int, cin: int, dil: int = 1, pad: int = 0, t_out: int | None = None, act=None,
               residual=None, out=None):
    """Stride-1 convolution over time, channels-last: x [B, T, ldx >= cin] bf16 -> [B, t_out, Cout8].
    ``pad`` input steps of zeros precede the signal (causal: (k-1)*dil, "same": (k-1)*dil // 2); reads
    past the end are zeros too.  On the GPU this is the implicit GEMM of csrc/gemm_sm100.cu (1-D mode)."""
    B, T, ldx = x.shape
    t_out = T if t_out is None else t_out
    cout8 = w_packed.shape[0]
    if not x.is_cuda:
        y = conv1d_nlc_reference(x, w_packed, bias, k, cin, dil, pad, t_out, act, residual).to(x.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    assert x.dtype == torch.bfloat16 and w_packed.dtype == torch.bfloat16 and x.stride(2) == 1 and x.stride(1) % 8 == 0
    if out is None:
        out = torch.empty(B, t_out, cout8, dtype=x.dtype, device=x.device)
    assert out.is_contiguous() or (out.stride(2) == 1 and out.stride(0) == t_out * out.stride(1))
    if residual is not None:
        assert residual.stride(-1) == 1 and residual.shape[0] == B and residual.shape[1] == t_out
        assert B == 1 or residual.stride(0) == t_out * residual.stride(1)
    st = nv.status_word(x.device)
    rc = nv.lib("gemm_sm100").omni_conv1d_nlc_bf16(
        nv.ptr(x), c_long(x.stride(1)), c_long(x.stride(0)), nv.ptr(w_packed), nv.ptr(out), c_int(out.stride(1)), c_int(B),
        c_int(T), c_int(t_out), c_int(cin), c_int(cout8), c_int(k), c_int(dil), c_int(pad), nv.ptr(bias), nv.ptr(residual),
        c_int(residual.stride(1) if residual is not None else 0), c_int(ACT[act]), nv.ptr(st), nv.stream_ptr())
    nv.check_rc(rc, "omni_conv1d_nlc_bf16")
    return out


def pack_conv_transpose1d_weight(w: torch.Tensor, bias: torch.Tensor | None, stride: int, padding: int = 0,
                                 dtype=torch.bfloat16):
    """Weights of ``ConvTranspose1d`` ([Cin, Cout, k], stride r, ``padding`` samples cut from the left
    end) re-stacked by output phase so that ONE stride-1 convolution produces all r phases at once:
    output sample t = q*r + phi is  sum_m x[q + d_phi - m] W[:, :, phi' + m*r]  with
    phi' = (phi + padding) % r, d_phi = (phi + padding) // r.  Returns (packed [r*Cout8, K*cin_pad],
    bias [r*Cout8], K taps, pad) for ``conv1d_nlc`` (tap j reads x[q + j - pad]); the convolution's
    [B, Tq, r*Cout8] result, read as [B, Tq*r, Cout8], is the transposed convolution."""
    Cin, Cout, k = w.shape
    r = stride
    cin_pad, cout8 = (Cin + 63) // 64 * 64, (Cout + 7) // 8 * 8
    offs = []
    for phi in range(r):
        pp, d = (phi + padding) % r, (phi + padding) // r
        m = 0
        while pp + m * r < k:
            offs.append((phi, d - m, pp + m * r))
            m += 1
    lo, hi = min(o for _, o, _ in offs), max(o for _, o, _ in offs)
    K, pad = hi - lo + 1, -lo
    p = torch.zeros(r, cout8, K, cin_pad, dtype=dtype, device=w.device)
    for phi, o, j in offs:
        p[phi, :Cout, o + pad, :Cin] = w[:, :, j].t().to(dtype)
    b = torch.zeros(r, cout8, dtype=dtype, device=w.device)
    if bias is not None:
        b[:, :Cout] = bias.to(dtype)
    return p.reshape(r * cout8, -1).contiguous(), b.reshape(-1).contiguous(), K, pad


def conv_transpose1d_nlc(x, packed, cin: int, stride: int, t_out: int, act=None):
    """x [B, T, >=cin] -> [B, t_out, Cout8]: ``packed`` from ``pack_conv_transpose1d_weight``; ``t_out`` is
    the number of output samples kept (counted after the left ``padding`` cut)."""
    w, b, K, pad = packed
    Tq = -(-t_out // stride)
    y = conv1d_nlc(x, w, b, K, cin, 1, pad, t_out=Tq, act=act)
    B = x.shape[0]
    y = y.view(B, Tq * stride, -1)
    return y if Tq * stride == t_out else y[:, :t_out].contiguous()


def snake_nlc(x, a, inv_b, out=None):
    """x + inv_b[c] * sin^2(x * a[c]) over the last (channel) dimension; a / inv_b fp32 [C]."""
    C = x.shape[-1]
    if not x.is_cuda:
        xf = x.float()
        y = (xf + inv_b.float() * torch.sin(xf * a.float()).pow(2)).to(x.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    assert x.dtype == torch.bfloat16 and x.is_contiguous() and C % 8 == 0 and a.dtype == torch.float32 and inv_b.dtype == torch.float32
    if out is None:
        out = torch.empty_like(x)
    rc = nv.lib("vae_ops").omni_snake_nlc(nv.ptr(x), c_long(C), nv.ptr(a), nv.ptr(inv_b), nv.ptr(out), c_long(C),
                                          c_long(x.numel() // C), c_int(C), nv.stream_ptr())
    nv.check_rc(rc, "omni_snake_nlc")
    return out


def dwconv1d_nlc(x, w_kc, bias, k: int, dil: int = 1, pad: int = 0):
    """Depthwise convolution over time, channels-last: x [B, T, C], w_kc fp32 [k, C], bias fp32 [C] or None."""
    B, T, C = x.shape
    if not x.is_cuda:
        xp = F.pad(x.float().transpose(1, 2), (pad, max(0, (k - 1) * dil - pad)))
        y = F.conv1d(xp, w_kc.float().t()[:, None, :], None if bias is None else bias.float(), dilation=dil, groups=C)
        return y[..., :T].transpose(1, 2).to(x.dtype)
    assert x.dtype == torch.bfloat16 and x.is_contiguous() and C % 8 == 0 and w_kc.dtype == torch.float32 and w_kc.is_contiguous()
    out = torch.empty_like(x)
    rc = nv.lib("vae_ops").omni_dwconv1d_nlc(nv.ptr(x), nv.ptr(w_kc), nv.ptr(bias), nv.ptr(out), c_int(B), c_int(T), c_int(C),
                                             c_int(k), c_int(dil), c_int(pad), nv.stream_ptr())
    nv.check_rc(rc, "omni_dwconv1d_nlc")
    return out


def aa_snake_nlc_reference(x, a, inv_b, up_filter, down_filter):
    """The anti-aliased snake of BigVGAN restated with PyTorch ops (x [B, T, C]): replicate-pad, 2x
    transposed-convolution up-sampling with ``up_filter`` [12], snake, replicate-pad, stride-2 convolution
    with ``down_filter`` [12]."""
    B, T, C = x.shape
    k = up_filter.numel()
    pad = k // 2 - 1
    xc = x.float().transpose(1, 2)
    y = F.pad(xc, (pad, pad), mode="replicate")
    y = 2 * F.conv_transpose1d(y, up_filter.float().view(1, 1, k).expand(C, -1, -1), stride=2, groups=C)
    pl, pr = pad * 2 + (k - 2) // 2, pad * 2 + (k - 2 + 1) // 2
    y = y[..., pl:-pr]
    y = y + inv_b.float()[None, :, None] * torch.sin(y * a.float()[None, :, None]).pow(2)
    y = F.pad(y, (k // 2 - (1 - k % 2), k // 2), mode="replicate")
    y = F.conv1d(y, down_filter.float().view(1, 1, k).expand(C, -1, -1), stride=2, groups=C)
    return y.transpose(1, 2)


def aa_snake_nlc(x, a, inv_b, up_filter, down_filter):
    """Up-sample x2, snake, down-sample x2 in one kernel (csrc/vae_ops.cu ``omni_aa_snake_nlc``); x [B, T, C]
    bf16 contiguous, a / inv_b fp32 [C], filters fp32 [12]."""
    if not x.is_cuda:
        return aa_snake_nlc_reference(x, a, inv_b, up_filter, down_filter).to(x.dtype)
    B, T, C = x.shape
    assert x.dtype == torch.bfloat16 and x.is_contiguous() and C % 8 == 0 and up_filter.numel() == 12 and down_filter.numel() == 12
    out = torch.empty_like(x)
    rc = nv.lib("vae_ops").omni_aa_snake_nlc(nv.ptr(x), nv.ptr(a), nv.ptr(inv_b), nv.ptr(up_filter), nv.ptr(down_filter),
                                             nv.ptr(out), c_int(B), c_int(T), c_int(C), nv.stream_ptr())
    nv.check_rc(rc, "omni_aa_snake_nlc")
    return out


def softmax_rows_(x: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """x [rows, N] bf16 (row pitch a multiple of 8 elements) <- softmax(scale * x) along the last dim, in place
    (csrc/vae_ops.cu ``omni_softmax_rows``)."""
    if not x.is_cuda:
        x.copy_(torch.softmax(x.float() * scale, dim=-1))
        return x
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
    rc = nv.lib("vae_ops").omni_softmax_rows(nv.ptr(x), ctypes.c_long(x.stride(0)), ctypes.c_long(x.shape[0]),
                                             c_int(x.shape[1]), ctypes.c_float(scale), nv.stream_ptr())
    nv.check_rc(rc, "omni_softmax_rows")
    return x


def wide_head_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, chunk_rows: int = 4096) -> torch.Tensor:
    """One attention head whose width is the channel count (the VAE mid block: 384 or 512), which the flash
    kernel's head sizes do not cover.  q, k, v: [B, N, C] bf16 views with the last dim contiguous.  On a GPU:
    scores = q k^T on the tcgen05 GEMM for ``chunk_rows`` queries at a time, row softmax in place, P v on the
    GEMM again against v transposed once; the score block (chunk_rows x N bf16) is the only scratch."""
    B, N, C = q.shape
    scale = C ** -0.5
    if not q.is_cuda or q.dtype != torch.bfloat16 or N % 8 or C % 8:
        return F.scaled_dot_product_attention(q[:, None], k[:, None], v[:, None])[:, 0]
    from .gemm import linear
    out = torch.empty(B, N, C, dtype=q.dtype, device=q.device)
    rows = min(chunk_rows, N)
    scores = torch.empty(rows, N, dtype=q.dtype, device=q.device)
    for b in range(B):
        vt = v[b].t().contiguous()
        for r0 in range(0, N, rows):
            n = min(rows, N - r0)
            s = scores[:n]
            linear(q[b, r0:r0 + n], k[b], out=s)
            softmax_rows_(s, scale)
            linear(s, vt, out=out[b, r0:r0 + n])
    return out


GN_SPLITS = 128          # partial sums per (sample, group) in the native kernel


def groupnorm_nhwc(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, groups: int, eps: float = 1e-6,
                   silu: bool = True, out: torch.Tensor | None = None) -> torch.Tensor:
    """GroupNorm over (pixels, channels of a group) per sample, then SiLU; x [N, H, W, C] channels-last (pitch >= C),
    gamma / beta fp32 [C] (csrc/vae_ops.cu ``omni_groupnorm_nhwc``: per-group sums in a fixed order, then one
    normalise-scale-shift-activate pass)."""
    N, H, W, ld = x.shape
    Cn = gamma.numel()
    if not x.is_cuda:
        xf = x[..., :Cn].float().permute(0, 3, 1, 2)
        y = F.group_norm(xf, groups, gamma.float(), beta.float(), eps)
        y = (F.silu(y) if silu else y).permute(0, 2, 3, 1).to(x.dtype)
        if out is not None:
            out[..., :Cn].copy_(y)
            return out
        return y.contiguous()
    assert x.dtype == torch.bfloat16 and x.is_contiguous() and gamma.dtype == torch.float32 and beta.dtype == torch.float32
    if out is None:
        out = torch.empty(N, H, W, Cn, dtype=x.dtype, device=x.device)
    partial = torch.empty(N * groups * GN_SPLITS * 2, dtype=torch.float32, device=x.device)
    rc = nv.lib("vae_ops").omni_groupnorm_nhwc(nv.ptr(x), c_long(ld), nv.ptr(out), c_long(out.stride(2)), c_int(N), c_long(H * W),
                                               c_int(Cn), c_int(groups), nv.ptr(gamma), nv.ptr(beta), ctypes.c_float(eps),
                                               c_int(1 if silu else 0), nv.ptr(partial), nv.stream_ptr())
    nv.check_rc(rc, "omni_groupnorm_nhwc")
    return out
