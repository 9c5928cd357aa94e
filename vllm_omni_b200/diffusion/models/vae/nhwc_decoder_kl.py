"""Channels-last execution of the 2-D ``AutoencoderKL`` decoder (FLUX / SD3 / Z-Image / BAGEL family: GroupNorm
ResNet blocks, one single-head attention in the mid block, nearest up-sampling) on the sm_100a kernels.

Built from a ``Decoder`` (same parameters, repacked once): every convolution is an implicit GEMM on the tcgen05
kernel with bias / residual in its epilogue, GroupNorm + SiLU is the two-kernel channels-last GroupNorm of
``ops.conv.groupnorm_nhwc``, the attention's q / k / v / out projections are 1x1 convolutions on the same kernel
around ``ops.conv.wide_head_attention`` (two GEMMs and a row softmax), activations stay NHWC bf16 from the latent
to the image.  Replaces the cuDNN path the reference takes through diffusers' ``AutoencoderKL``
(vllm_omni/diffusion/models/flux/pipeline_flux.py, the ``vae.decode`` call).
"""
from __future__ import annotations

import torch

from ....ops import conv as C


class _Conv:
    def __init__(self, weight4d: torch.Tensor, bias, dtype):
        self.k = weight4d.shape[-1]
        self.cin, self.cout = weight4d.shape[1], weight4d.shape[0]
        self.w, self.b = C.pack_conv_weight(weight4d, bias, dtype)

    @classmethod
    def of(cls, m, dtype):
        if isinstance(m, torch.nn.Linear):                     # a Linear over channels is a 1x1 convolution
            return cls(m.weight.data[:, :, None, None], m.bias.data if m.bias is not None else None, dtype)
        return cls(m.weight.data, m.bias.data if m.bias is not None else None, dtype)

    def __call__(self, x, residual=None):
        return C.conv2d_nhwc(x, self.w, self.b, self.k, self.cin, residual=residual)


class _Norm:
    def __init__(self, m: torch.nn.GroupNorm):
        self.g, self.eps = m.num_groups, m.eps
        self.gamma, self.beta = m.weight.data.float().contiguous(), m.bias.data.float().contiguous()

    def __call__(self, x, silu=True):
        return C.groupnorm_nhwc(x, self.gamma, self.beta, self.g, self.eps, silu=silu)


class NHWCDecoderKL:
    @staticmethod
    def supported(decoder) -> bool:
        """The native GroupNorm wants C / 8 to divide 256 and at most 64 groups; other geometries keep the cuDNN path."""
        for m in decoder.modules():
            if isinstance(m, torch.nn.GroupNorm):
                c = m.num_channels
                if c % 8 or 256 % (c // 8) or c // 8 > 256 or m.num_groups > 64:
                    return False
        return True

    def __init__(self, decoder, post_quant_conv=None, dtype=torch.bfloat16):
        d = decoder
        self.dtype = dtype
        self.post_quant = _Conv.of(post_quant_conv, dtype) if post_quant_conv is not None else None
        self.conv_in = _Conv.of(d.conv_in, dtype)
        self.stages = []

        def res(m):
            self.stages.append(("res", _Norm(m.norm1), _Conv.of(m.conv1, dtype), _Norm(m.norm2), _Conv.of(m.conv2, dtype),
                                _Conv.of(m.conv_shortcut, dtype) if m.conv_shortcut is not None else None))
        res(d.mid_block.resnets[0])
        for a in d.mid_block.attentions:
            w = torch.cat([a.to_q.weight.data, a.to_k.weight.data, a.to_v.weight.data], 0)[:, :, None, None]
            b = torch.cat([a.to_q.bias.data, a.to_k.bias.data, a.to_v.bias.data], 0)
            self.stages.append(("attn", _Norm(a.group_norm), _Conv(w, b, dtype), _Conv.of(a.to_out[0], dtype), a.to_q.out_features))
        res(d.mid_block.resnets[1])
        for blk in d.up_blocks:
            for r in blk.resnets:
                res(r)
            if blk.upsamplers is not None:
                self.stages.append(("up", _Conv.of(blk.upsamplers[0].conv, dtype)))
        self.norm_out = _Norm(d.conv_norm_out)
        self.conv_out = _Conv.of(d.conv_out, dtype)

    @torch.no_grad()
    def __call__(self, z: torch.Tensor) -> torch.Tensor:
        """z: [B, C, h, w] model-space latents -> [B, 3, 8h, 8w] fp32 in [-1, 1]."""
        x = C.nchw_to_nhwc(z, dtype=self.dtype)
        if self.post_quant is not None:
            x = self.post_quant(x)
        x = self.conv_in(x)
        for st in self.stages:
            if st[0] == "res":
                _, n1, c1, n2, c2, sc = st
                h = c1(n1(x))
                skip = x if sc is None else sc(x)
                x = c2(n2(h), residual=skip)
            elif st[0] == "attn":
                _, gn, qkv, proj, ch = st
                B, H, W, _ = x.shape
                t = qkv(gn(x, silu=False)).view(B, H * W, 3, ch)
                o = C.wide_head_attention(t[:, :, 0], t[:, :, 1], t[:, :, 2])
                x = proj(o.reshape(B, H, W, ch).contiguous(), residual=x)
            else:
                x = st[1](C.upsample2x_nhwc(x))
        x = self.conv_out(self.norm_out(x))
        return C.nhwc_to_image(x)
