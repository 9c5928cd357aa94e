"""Channels-last execution of the image VAE decoder on the sm_100a kernels.

Built from a ``Decoder2d`` (same parameters, repacked once): every convolution is an implicit
GEMM on the tcgen05 kernel with bias / residual in its epilogue, RMS-norm + SiLU is one fused
kernel per pixel row, activations stay NHWC bf16 from the latent to the image.  The single
mid-block attention (one head of width C, outside the flash kernel's head sizes) is two GEMMs on the
same kernel around a row-softmax kernel (``ops.conv.wide_head_attention``).  Replaces the cuDNN path the
reference takes through diffusers (vllm_omni/diffusion/models/qwen_image/
autoencoder_kl_qwenimage.py).
"""
from __future__ import annotations

import torch

from ....ops import conv as C


class _Conv:
    def __init__(self, m: torch.nn.Conv2d, dtype):
        self.k = m.kernel_size[0]
        self.cin, self.cout = m.in_channels, m.out_channels
        self.w, self.b = C.pack_conv_weight(m.weight.data, m.bias.data if m.bias is not None else None, dtype)

    def __call__(self, x, act=None, residual=None):
        return C.conv2d_nhwc(x, self.w, self.b, self.k, self.cin, act=act, residual=residual)


class NHWCDecoder:
    def __init__(self, decoder, post_quant_conv=None, dtype=torch.bfloat16):
        d = decoder
        g = lambda n: n.gamma.data.to(dtype).contiguous()
        self.dtype = dtype
        self.post_quant = _Conv(post_quant_conv, dtype) if post_quant_conv is not None else None
        self.conv_in = _Conv(d.conv_in, dtype)
        self.stages = []
        for m in list(d.mid) + [m for blk in d.up_blocks for m in blk]:
            name = type(m).__name__
            if name == "ResBlock":
                self.stages.append(("res", g(m.norm1), _Conv(m.conv1, dtype), g(m.norm2), _Conv(m.conv2, dtype),
                                    _Conv(m.shortcut, dtype) if m.shortcut is not None else None))
            elif name == "AttnBlock":
                self.stages.append(("attn", g(m.norm), _Conv(m.to_qkv, dtype), _Conv(m.proj, dtype)))
            elif name == "Upsample":
                self.stages.append(("up", _Conv(m.conv, dtype)))
            else:
                raise TypeError(f"unexpected decoder block {name}")
        self.norm_out = g(d.norm_out)
        self.conv_out = _Conv(d.conv_out, dtype)

    @torch.no_grad()
    def __call__(self, z: torch.Tensor, uint8: bool = False) -> torch.Tensor:
        """z: [B, z_dim, h, w] de-normalised latents -> [B, 3, 8h, 8w] fp32 in [-1, 1] (or uint8 NHWC)."""
        x = C.nchw_to_nhwc(z, dtype=self.dtype)
        if self.post_quant is not None:
            x = self.post_quant(x)
        x = self.conv_in(x)
        for st in self.stages:
            if st[0] == "res":
                _, g1, c1, g2, c2, sc = st
                h = c1(C.rmsnorm_silu_nhwc(x, g1))
                skip = x if sc is None else sc(x)
                x = c2(C.rmsnorm_silu_nhwc(h, g2), residual=skip)
            elif st[0] == "attn":
                _, gn, qkv, proj = st
                B, H, W, ch = x.shape
                t = qkv(C.rmsnorm_silu_nhwc(x, gn, silu=False)).view(B, H * W, 3, ch)
                o = C.wide_head_attention(t[:, :, 0], t[:, :, 1], t[:, :, 2])
                x = proj(o.reshape(B, H, W, ch).contiguous(), residual=x)
            else:
                x = st[1](C.upsample2x_nhwc(x))
        x = self.conv_out(C.rmsnorm_silu_nhwc(x, self.norm_out))
        return C.nhwc_to_image(x, uint8=uint8)
