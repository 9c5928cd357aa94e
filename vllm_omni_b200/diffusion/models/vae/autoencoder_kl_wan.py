"""Causal 3-D VAE decoder (Wan 2.1 / Qwen-Image family) for video latents.

[B, 16, T, h, w] -> [B, 3, 1 + 4 (T - 1), 8h, 8w].  Every convolution is causal in time
(front padding only), so frame t never sees later frames; the temporal up-sampling layers
double the frame count except for the first frame
(vllm_omni/diffusion/models/qwen_image/autoencoder_kl_qwenimage.py, diffusers AutoencoderKLWan).
Latent frames are decoded in a streaming fashion: each causal convolution keeps the last two
input frames of the previous chunk (``feat cache``), so memory is bounded by one chunk and the
result equals the full-clip decode.  Spatially the clip can be split into overlapping tiles
across ranks (parallel/vae_patch_parallel.py).

On a GPU with the module in bf16 the decoder runs channels-last on this library's kernels
(``nhwc_video_decoder.NHWCVideoDecoder``: every causal 3-D convolution as kT launches of the 2-D
implicit-GEMM kernel accumulating through its residual operand); ``OMNI_VAE_IMPL=torch`` or an fp32
module keeps the cuDNN path below.
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F
from torch import nn

from .autoencoder_kl_qwenimage import QwenImageVAEConfig


class CausalConv3d(nn.Conv3d):
    """3-D convolution with causal time padding and an optional per-layer frame cache."""

    def __init__(self, cin, cout, k, padding=0, **kw):
        k = (k, k, k) if isinstance(k, int) else k
        p = (padding,) * 3 if isinstance(padding, int) else padding
        super().__init__(cin, cout, k, padding=0, **kw)
        self._pad = (p[2], p[2], p[1], p[1], 2 * p[0], 0)
        self._tpad = 2 * p[0]

    def forward(self, x, cache: dict | None = None, key=None):
        pad = list(self._pad)
        if cache is not None and self._tpad > 0:
            prev = cache.get(key)
            cache[key] = x[:, :, -self._tpad:].clone() if x.shape[2] >= self._tpad else (
                torch.cat([prev[:, :, -(self._tpad - x.shape[2]):], x], 2) if prev is not None else x.clone())
            if prev is not None:
                x = torch.cat([prev, x], dim=2)
                pad[4] = max(0, self._tpad - prev.shape[2])
        return super().forward(F.pad(x, pad))


class RMSNorm3d(nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.gamma = nn.Parameter(torch.ones(dim))
        self.scale = dim ** 0.5

    def forward(self, x):
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).sum(1, keepdim=True).clamp_min(1e-24)) * self.scale
        return (y * self.gamma.float().view(1, -1, 1, 1, 1)).to(x.dtype)


class ResBlock3d(nn.Module):
    def __init__(self, cin, cout):
        super().__init__()
        self.norm1, self.conv1 = RMSNorm3d(cin), CausalConv3d(cin, cout, 3, padding=1)
        self.norm2, self.conv2 = RMSNorm3d(cout), CausalConv3d(cout, cout, 3, padding=1)
        self.shortcut = CausalConv3d(cin, cout, 1) if cin != cout else None

    def forward(self, x, cache, key):
        h = self.conv1(F.silu(self.norm1(x)), cache, (key, 1))
        h = self.conv2(F.silu(self.norm2(h)), cache, (key, 2))
        return h + (x if self.shortcut is None else self.shortcut(x))


class AttnBlock3d(nn.Module):
    """Per-frame single-head spatial attention."""

    def __init__(self, dim):
        super().__init__()
        self.norm = RMSNorm3d(dim)
        self.to_qkv = nn.Conv2d(dim, 3 * dim, 1)
        self.proj = nn.Conv2d(dim, dim, 1)

    def forward(self, x, cache=None, key=None):
        B, C, T, H, W = x.shape
        y = self.norm(x).permute(0, 2, 1, 3, 4).reshape(B * T, C, H, W)
        qkv = self.to_qkv(y).reshape(B * T, 3, C, H * W).permute(1, 0, 3, 2)
        o = F.scaled_dot_product_attention(qkv[0][:, None], qkv[1][:, None], qkv[2][:, None])[:, 0]
        o = self.proj(o.permute(0, 2, 1).reshape(B * T, C, H, W)).view(B, T, C, H, W).permute(0, 2, 1, 3, 4)
        return x + o


class Upsample3d(nn.Module):
    def __init__(self, dim, temporal: bool):
        super().__init__()
        self.conv = nn.Conv2d(dim, dim // 2, 3, padding=1)
        self.time_conv = CausalConv3d(dim, 2 * dim, (3, 1, 1), padding=(1, 0, 0)) if temporal else None

    def forward(self, x, cache, key):
        B, C, T, H, W = x.shape
        if self.time_conv is not None:
            first = cache is None or not cache.get(("seen", key))
            if cache is not None:
                cache[("seen", key)] = True
            y = self.time_conv(x, cache, (key, "t"))                      # [B, 2C, T, H, W]
            y = y.view(B, 2, C, T, H, W).permute(0, 2, 3, 1, 4, 5).reshape(B, C, 2 * T, H, W)
            if first:                                                      # the very first frame is not doubled
                y = y[:, :, 1:]
            x = y
            T = x.shape[2]
        z = x.permute(0, 2, 1, 3, 4).reshape(B * T, C, H, W)
        z = self.conv(F.interpolate(z, scale_factor=2.0, mode="nearest-exact"))
        return z.view(B, T, C // 2, 2 * H, 2 * W).permute(0, 2, 1, 3, 4)


class WanDecoder3d(nn.Module):
    def __init__(self, cfg: QwenImageVAEConfig):
        super().__init__()
        dims = [cfg.base_dim * m for m in [cfg.dim_mult[-1]] + list(cfg.dim_mult[::-1])]
        self.conv_in = CausalConv3d(cfg.z_dim, dims[0], 3, padding=1)
        self.mid = nn.ModuleList([ResBlock3d(dims[0], dims[0]), AttnBlock3d(dims[0]), ResBlock3d(dims[0], dims[0])])
        temporal = list(cfg.temperal_downsample[::-1])
        ups = []
        for i, (cin, cout) in enumerate(zip(dims[:-1], dims[1:])):
            if i > 0:
                cin = cin // 2
            blk = [ResBlock3d(cin if j == 0 else cout, cout) for j in range(cfg.num_res_blocks + 1)]
            if i != len(cfg.dim_mult) - 1:
                blk.append(Upsample3d(cout, temporal[i] if i < len(temporal) else False))
            ups.append(nn.ModuleList(blk))
        self.up_blocks = nn.ModuleList(ups)
        self.norm_out = RMSNorm3d(dims[-1])
        self.conv_out = CausalConv3d(dims[-1], 3, 3, padding=1)

    def forward(self, z, cache=None):
        x = self.conv_in(z, cache, "in")
        for i, m in enumerate(self.mid):
            x = m(x, cache, ("mid", i))
        for bi, blk in enumerate(self.up_blocks):
            for mi, m in enumerate(blk):
                x = m(x, cache, ("up", bi, mi))
        return self.conv_out(F.silu(self.norm_out(x)), cache, "out")


class AutoencoderKLWan(nn.Module):
    def __init__(self, cfg: QwenImageVAEConfig | None = None):
        super().__init__()
        self.cfg = cfg = cfg or QwenImageVAEConfig()
        self.post_quant_conv = CausalConv3d(cfg.z_dim, cfg.z_dim, 1)
        self.decoder = WanDecoder3d(cfg)
        self.decoder_impl = os.environ.get("OMNI_VAE_IMPL", "nhwc")      # "nhwc" (own kernels) | "torch" (cuDNN)
        self._nhwc = None

    @property
    def dtype(self):
        return self.post_quant_conv.weight.dtype

    def denormalize(self, z):
        mean = torch.tensor(self.cfg.latents_mean, device=z.device, dtype=z.dtype).view(1, -1, 1, 1, 1)
        std = torch.tensor(self.cfg.latents_std, device=z.device, dtype=z.dtype).view(1, -1, 1, 1, 1)
        return z * std + mean

    @torch.no_grad()
    def decode(self, z: torch.Tensor, chunk_frames: int = 1) -> torch.Tensor:
        """Streaming decode, ``chunk_frames`` latent frames at a time (0 = whole clip at once)."""
        if z.is_cuda and self.dtype == torch.bfloat16 and self.decoder_impl != "torch":
            if self._nhwc is None:
                from .nhwc_video_decoder import NHWCVideoDecoder
                self._nhwc = NHWCVideoDecoder(self.decoder, self.post_quant_conv, torch.bfloat16)
            return self._nhwc(self.denormalize(z.float()), chunk_frames)
        z = self.denormalize(z.float()).to(self.dtype)
        z = self.post_quant_conv(z)
        if chunk_frames <= 0 or z.shape[2] <= chunk_frames:
            return self.decoder(z, {}).clamp_(-1, 1)
        cache: dict = {}
        outs = []
        for t in range(0, z.shape[2], chunk_frames):
            outs.append(self.decoder(z[:, :, t:t + chunk_frames], cache))
        return torch.cat(outs, dim=2).clamp_(-1, 1)
