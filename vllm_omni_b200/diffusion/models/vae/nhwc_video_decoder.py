"""Channels-last execution of the causal 3-D (video) VAE decoder on the sm_100a kernels.

Built from a ``WanDecoder3d`` (same parameters, repacked once).  Activations are frames-major
channels-last bf16, ``[B, T, H, W, C]``.  A causal 3-D convolution with a ``kT x k x k`` kernel is ``kT``
launches of the 2-D implicit-GEMM kernel: tap ``j`` convolves the frames shifted by ``kT - 1 - j`` into the
past with the weight slice ``W[:, :, j]`` and accumulates into the same output through the kernel's residual
operand (the block's skip connection rides on the first tap), so the whole convolution is tensor-core GEMM
work with K = k*k*Cin per launch and no im2col.  RMS-norm + SiLU is one fused kernel per pixel row, the
per-frame mid-block attention is two GEMMs around a row softmax (``ops.conv.wide_head_attention``), nearest
up-sampling and the layout changes are this library's element-wise kernels.

Latent frames are decoded in chunks exactly like the PyTorch module does: every causal convolution keeps the
last ``kT - 1`` input frames of the previous chunk, so memory is bounded by one chunk and the result does not
depend on the chunking.  Replaces the cuDNN ``Conv3d`` path the reference takes through diffusers'
``AutoencoderKLWan`` (vllm_omni/diffusion/models/wan2_2/pipeline_wan2_2.py, the ``vae.decode`` call;
vllm_omni/diffusion/models/qwen_image/autoencoder_kl_qwenimage.py for the layer definitions).
"""
from __future__ import annotations

import torch

from ....ops import conv as C


class _CausalConv:
    """One causal convolution: per temporal tap a packed 2-D weight."""

    def __init__(self, m: torch.nn.Conv3d, dtype):
        kT, k, _ = m.kernel_size
        self.kT, self.k = kT, k
        self.cin, self.cout = m.in_channels, m.out_channels
        w = m.weight.data                                           # [Cout, Cin, kT, k, k]
        self.taps = []
        for j in range(kT):
            wj, bj = C.pack_conv_weight(w[:, :, j].contiguous(), m.bias.data if (m.bias is not None and j == 0) else None, dtype)
            self.taps.append((wj, bj))

    def __call__(self, x: torch.Tensor, cache: dict | None, key, residual: torch.Tensor | None = None) -> torch.Tensor:
        """x [B, T, H, W, Cin8] -> [B, T, H, W, Cout8]; ``residual`` (same shape as the result) is added."""
        B, T, H, W, ld = x.shape
        past = self.kT - 1
        if past:
            prev = cache.get(key) if cache is not None else None
            if prev is None:
                prev = x.new_zeros(B, past, H, W, ld)                 # causal zero padding in front of the clip
            elif prev.shape[1] < past:
                prev = torch.cat([x.new_zeros(B, past - prev.shape[1], H, W, ld), prev], dim=1)
            xin = torch.cat([prev, x], dim=1)
            if cache is not None:
                cache[key] = xin[:, -past:].clone()
        else:
            xin = x
        out = None
        for j, (wj, bj) in enumerate(self.taps):
            frames = xin[:, j:j + T]
            frames = frames.reshape(B * T, H, W, ld) if B == 1 else frames.contiguous().view(B * T, H, W, ld)
            if not frames.is_contiguous():
                frames = frames.contiguous()
            res = out if j > 0 else (residual.reshape(B * T, H, W, -1) if residual is not None else None)
            out = C.conv2d_nhwc(frames, wj, bj, self.k, self.cin, residual=res, out=out)
        return out.view(B, T, H, W, -1)


class _Conv2dFrames:
    """A 2-D convolution applied to every frame."""

    def __init__(self, m: torch.nn.Conv2d, dtype):
        self.k, self.cin = m.kernel_size[0], m.in_channels
        self.w, self.b = C.pack_conv_weight(m.weight.data, m.bias.data if m.bias is not None else None, dtype)

    def __call__(self, x, residual=None):
        return C.conv2d_nhwc(x, self.w, self.b, self.k, self.cin, residual=residual)


class NHWCVideoDecoder:
    def __init__(self, decoder, post_quant_conv=None, dtype=torch.bfloat16):
        d = decoder
        g = lambda n: n.gamma.data.to(dtype).contiguous()
        self.dtype = dtype
        self.post_quant = _CausalConv(post_quant_conv, dtype) if post_quant_conv is not None else None
        self.conv_in = _CausalConv(d.conv_in, dtype)
        self.stages = []
        mods = [(("mid", i), m) for i, m in enumerate(d.mid)] + \
               [(("up", bi, mi), m) for bi, blk in enumerate(d.up_blocks) for mi, m in enumerate(blk)]
        for key, m in mods:
            name = type(m).__name__
            if name == "ResBlock3d":
                self.stages.append(("res", key, g(m.norm1), _CausalConv(m.conv1, dtype), g(m.norm2), _CausalConv(m.conv2, dtype),
                                    _CausalConv(m.shortcut, dtype) if m.shortcut is not None else None))
            elif name == "AttnBlock3d":
                self.stages.append(("attn", key, g(m.norm), _Conv2dFrames(m.to_qkv, dtype), _Conv2dFrames(m.proj, dtype)))
            elif name == "Upsample3d":
                self.stages.append(("up", key, _Conv2dFrames(m.conv, dtype),
                                    _CausalConv(m.time_conv, dtype) if m.time_conv is not None else None))
            else:
                raise TypeError(f"unexpected decoder block {name}")
        self.norm_out = g(d.norm_out)
        self.conv_out = _CausalConv(d.conv_out, dtype)

    def _chunk(self, x: torch.Tensor, cache: dict) -> torch.Tensor:
        """x [B, T, h, w, C8] latent frames (already through the post-quant convolution) -> [B, T', 8h, 8w, 8]."""
        x = self.conv_in(x, cache, "in")
        for st in self.stages:
            kind, key = st[0], st[1]
            if kind == "res":
                _, _, g1, c1, g2, c2, sc = st
                h = c1(C.rmsnorm_silu_nhwc(x, g1), cache, (key, 1))
                skip = x if sc is None else sc(x, cache, (key, "s"))
                x = c2(C.rmsnorm_silu_nhwc(h, g2), cache, (key, 2), residual=skip)
            elif kind == "attn":
                _, _, gn, qkv, proj = st
                B, T, H, W, ch = x.shape
                xf = x.view(B * T, H, W, ch)
                t = qkv(C.rmsnorm_silu_nhwc(xf, gn, silu=False)).view(B * T, H * W, 3, -1)[..., :ch]
                o = C.wide_head_attention(t[:, :, 0], t[:, :, 1], t[:, :, 2])
                x = proj(o.view(B * T, H, W, ch), residual=xf).view(B, T, H, W, -1)
            else:
                _, _, conv, tconv = st
                B, T, H, W, ch = x.shape
                if tconv is not None:
                    first = not cache.get(("seen", key))
                    cache[("seen", key)] = True
                    y = tconv(x, cache, (key, "t"))                                      # [B, T, H, W, 2C]
                    y = y[..., :2 * ch].view(B, T, H, W, 2, ch).permute(0, 1, 4, 2, 3, 5).reshape(B, 2 * T, H, W, ch)
                    x = y[:, 1:] if first else y                                          # the very first frame is not doubled
                    T = x.shape[1]
                z = C.upsample2x_nhwc(x.reshape(B * T, H, W, ch).contiguous())
                x = conv(z).view(B, T, 2 * H, 2 * W, -1)
        return self.conv_out(C.rmsnorm_silu_nhwc(x, self.norm_out), cache, "out")

    @torch.no_grad()
    def __call__(self, z: torch.Tensor, chunk_frames: int = 1) -> torch.Tensor:
        """z: [B, z_dim, T, h, w] de-normalised latents -> [B, 3, T', 8h, 8w] fp32 in [-1, 1]."""
        B, Cz, T, h, w = z.shape
        x = C.nchw_to_nhwc(z.permute(0, 2, 1, 3, 4).reshape(B * T, Cz, h, w).contiguous(), dtype=self.dtype)
        x = x.view(B, T, h, w, -1)
        cache: dict = {}
        if self.post_quant is not None:
            x = self.post_quant(x, None, None)
        step = T if chunk_frames <= 0 else chunk_frames
        outs = []
        for t in range(0, T, step):
            y = self._chunk(x[:, t:t + step].contiguous(), cache)                        # [B, T', H, W, 8]
            Bt, Tt, H, W, ld = y.shape
            img = C.nhwc_to_image(y.reshape(Bt * Tt, H, W, ld))                           # [B*T', 3, H, W] fp32, clamped
            outs.append(img.view(Bt, Tt, 3, H, W).permute(0, 2, 1, 3, 4))
        return torch.cat(outs, dim=2)
