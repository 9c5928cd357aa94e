"""Image-mode decoder/encoder of the Qwen-Image / Wan-2.1 causal-3D VAE.

For a single frame every causal 3-D convolution of ``AutoencoderKLQwenImage``
(vllm_omni/diffusion/models/qwen_image/autoencoder_kl_qwenimage.py) sees only zero
padding in time, so it equals a 2-D convolution with the LAST temporal slice of its
kernel, and the temporal up/down-sampling convolutions are skipped for the first frame.
This module is that 2-D network; ``load_weights`` slices 5-D checkpoint kernels.  The
video (multi-frame) path lives in ``autoencoder_kl_wan.py``.

Layout: channels_last bf16 so the convolutions run as implicit GEMMs on tensor cores.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ....ops.conv import wide_head_attention


@dataclass
class QwenImageVAEConfig:
    base_dim: int = 96
    z_dim: int = 16
    dim_mult: tuple = (1, 2, 4, 4)
    num_res_blocks: int = 2
    temperal_downsample: tuple = (False, True, True)
    latents_mean: tuple = (-0.7571, -0.7089, -0.9113, 0.1075, -0.1745, 0.9653, -0.1517, 1.5508,
                           0.4134, -0.0715, 0.5517, -0.3632, -0.1922, -0.9497, 0.2503, -0.2921)
    latents_std: tuple = (2.8184, 1.4541, 2.3275, 2.6558, 1.2196, 1.7708, 2.6052, 2.0743,
                          3.2687, 2.1526, 2.8652, 1.5579, 1.6382, 1.1253, 2.8251, 1.9160)

    @property
    def spatial_scale(self) -> int:
        return 2 ** (len(self.dim_mult) - 1)

    @classmethod
    def from_dict(cls, d):
        keys = set(cls.__dataclass_fields__)
        return cls(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in d.items() if k in keys})


class RMSNorm2d(nn.Module):
    """F.normalize over channels * sqrt(C) * gamma (the VAE's ``RMS_norm``)."""

    def __init__(self, dim):
        super().__init__()
        self.gamma = nn.Parameter(torch.ones(dim))
        self.scale = dim ** 0.5

    def forward(self, x):
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).sum(1, keepdim=True).clamp_min(1e-24)) * self.scale
        return (y * self.gamma.float().view(1, -1, 1, 1)).to(x.dtype)


class ResBlock(nn.Module):
    def __init__(self, cin, cout):
        super().__init__()
        self.norm1, self.conv1 = RMSNorm2d(cin), nn.Conv2d(cin, cout, 3, padding=1)
        self.norm2, self.conv2 = RMSNorm2d(cout), nn.Conv2d(cout, cout, 3, padding=1)
        self.shortcut = nn.Conv2d(cin, cout, 1) if cin != cout else None

    def forward(self, x):
        h = self.conv1(F.silu(self.norm1(x)))
        h = self.conv2(F.silu(self.norm2(h)))
        return h + (x if self.shortcut is None else self.shortcut(x))


class AttnBlock(nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.norm = RMSNorm2d(dim)
        self.to_qkv = nn.Conv2d(dim, 3 * dim, 1)
        self.proj = nn.Conv2d(dim, dim, 1)

    def forward(self, x):
        B, C, H, W = x.shape
        qkv = self.to_qkv(self.norm(x)).reshape(B, 3, C, H * W).permute(1, 0, 3, 2).contiguous()   # 3, B, HW, C
        o = wide_head_attention(qkv[0], qkv[1], qkv[2])
        o = o.permute(0, 2, 1).reshape(B, C, H, W)
        return x + self.proj(o)


class Upsample(nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.conv = nn.Conv2d(dim, dim // 2, 3, padding=1)

    def forward(self, x):
        return self.conv(F.interpolate(x, scale_factor=2.0, mode="nearest-exact"))


class Downsample(nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.conv = nn.Conv2d(dim, dim, 3, stride=2)

    def forward(self, x):
        return self.conv(F.pad(x, (0, 1, 0, 1)))


class Decoder2d(nn.Module):
    def __init__(self, cfg: QwenImageVAEConfig):
        super().__init__()
        dims = [cfg.base_dim * m for m in [cfg.dim_mult[-1]] + list(cfg.dim_mult[::-1])]
        self.conv_in = nn.Conv2d(cfg.z_dim, dims[0], 3, padding=1)
        self.mid = nn.ModuleList([ResBlock(dims[0], dims[0]), AttnBlock(dims[0]), ResBlock(dims[0], dims[0])])
        ups = []
        for i, (cin, cout) in enumerate(zip(dims[:-1], dims[1:])):
            if i > 0:
                cin = cin // 2
            blk = [ResBlock(cin if j == 0 else cout, cout) for j in range(cfg.num_res_blocks + 1)]
            if i != len(cfg.dim_mult) - 1:
                blk.append(Upsample(cout))
            ups.append(nn.ModuleList(blk))
        self.up_blocks = nn.ModuleList(ups)
        self.norm_out = RMSNorm2d(dims[-1])
        self.conv_out = nn.Conv2d(dims[-1], 3, 3, padding=1)

    def forward(self, z):
        x = self.conv_in(z)
        for m in self.mid:
            x = m(x)
        for blk in self.up_blocks:
            for m in blk:
                x = m(x)
        return self.conv_out(F.silu(self.norm_out(x)))


class Encoder2d(nn.Module):
    def __init__(self, cfg: QwenImageVAEConfig):
        super().__init__()
        dims = [cfg.base_dim * m for m in [1] + list(cfg.dim_mult)]
        self.conv_in = nn.Conv2d(3, dims[0], 3, padding=1)
        downs = []
        for i, (cin, cout) in enumerate(zip(dims[:-1], dims[1:])):
            blk = [ResBlock(cin if j == 0 else cout, cout) for j in range(cfg.num_res_blocks)]
            if i != len(cfg.dim_mult) - 1:
                blk.append(Downsample(cout))
            downs.append(nn.ModuleList(blk))
        self.down_blocks = nn.ModuleList(downs)
        self.mid = nn.ModuleList([ResBlock(dims[-1], dims[-1]), AttnBlock(dims[-1]), ResBlock(dims[-1], dims[-1])])
        self.norm_out = RMSNorm2d(dims[-1])
        self.conv_out = nn.Conv2d(dims[-1], 2 * cfg.z_dim, 3, padding=1)

    def forward(self, x):
        x = self.conv_in(x)
        for blk in self.down_blocks:
            for m in blk:
                x = m(x)
        for m in self.mid:
            x = m(x)
        return self.conv_out(F.silu(self.norm_out(x)))


class AutoencoderKLQwenImage2d(nn.Module):
    def __init__(self, cfg: QwenImageVAEConfig | None = None, with_encoder: bool = False):
        super().__init__()
        self.cfg = cfg = cfg or QwenImageVAEConfig()
        self.post_quant_conv = nn.Conv2d(cfg.z_dim, cfg.z_dim, 1)
        self.decoder = Decoder2d(cfg)
        self.encoder = Encoder2d(cfg) if with_encoder else None
        self.quant_conv = nn.Conv2d(2 * cfg.z_dim, 2 * cfg.z_dim, 1) if with_encoder else None
        self.use_tiling = False
        self.tile_latent = 64
        self.tile_overlap = 8
        self.decoder_impl = os.environ.get("OMNI_VAE_IMPL", "nhwc")      # "nhwc" (own kernels) | "torch" (cuDNN)
        self._nhwc = None                                               # repacked weights, built on first use

    @property
    def dtype(self):
        return self.post_quant_conv.weight.dtype

    def denormalize(self, z):
        mean = torch.tensor(self.cfg.latents_mean, device=z.device, dtype=z.dtype).view(1, -1, 1, 1)
        std = torch.tensor(self.cfg.latents_std, device=z.device, dtype=z.dtype).view(1, -1, 1, 1)
        return z * std + mean

    def normalize(self, z):
        mean = torch.tensor(self.cfg.latents_mean, device=z.device, dtype=z.dtype).view(1, -1, 1, 1)
        std = torch.tensor(self.cfg.latents_std, device=z.device, dtype=z.dtype).view(1, -1, 1, 1)
        return (z - mean) / std

    @torch.no_grad()
    def decode(self, z):
        """z: [B, z_dim, h, w] normalised latents -> [B, 3, 8h, 8w] in [-1, 1]."""
        z = self.denormalize(z.float()).to(self.dtype)
        tiled = self.use_tiling and max(z.shape[-2:]) > self.tile_latent
        if z.is_cuda and self.dtype == torch.bfloat16 and not tiled and self.decoder_impl != "torch":
            # channels-last decoder on the implicit-GEMM convolution kernels
            if self._nhwc is None:
                from .nhwc_decoder import NHWCDecoder
                self._nhwc = NHWCDecoder(self.decoder, self.post_quant_conv, torch.bfloat16)
            return self._nhwc(z)
        if z.is_cuda:
            z = z.contiguous(memory_format=torch.channels_last)
        if tiled:
            return self._tiled_decode(z)
        return self.decoder(self.post_quant_conv(z)).clamp_(-1, 1)

    def _tiled_decode(self, z):
        """Overlapping latent tiles, linear blend across the overlaps (diffusers' tiled VAE)."""
        from ....parallel.vae_patch_parallel import blend_tiles, plan_tiles
        B, C, H, W = z.shape
        s = self.cfg.spatial_scale
        tiles = plan_tiles(H, W, self.tile_latent, self.tile_overlap)
        dec = [(t, self.decoder(self.post_quant_conv(z[:, :, t.y0:t.y1, t.x0:t.x1]))) for t in tiles]
        return blend_tiles(dec, H * s, W * s, s, self.tile_overlap * s).clamp_(-1, 1)

    @torch.no_grad()
    def encode(self, x, sample: bool = False, generator=None):
        assert self.encoder is not None, "VAE was built without an encoder"
        h = self.quant_conv(self.encoder(x.to(self.dtype)))
        mean, logvar = h.float().chunk(2, dim=1)
        if sample:
            mean = mean + torch.exp(0.5 * logvar.clamp(-30, 20)) * torch.randn(
                mean.shape, generator=generator, device=mean.device)
        return self.normalize(mean)

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        """Accepts diffusers ``AutoencoderKLQwenImage`` names; 5-D kernels are sliced to 2-D."""
        self._nhwc = None
        own = dict(self.named_parameters())
        loaded = set()
        for name, w in weights:
            tgt = _map_vae_name(name)
            if tgt is None or tgt not in own:
                continue
            p = own[tgt]
            if w.dim() == 5:
                w = w[:, :, -1]
            if w.dim() == 3 and p.dim() == 1:      # gamma stored as [C,1,1]
                w = w.reshape(-1)
            if w.dim() == 4 and p.dim() == 1:
                w = w.reshape(-1)
            p.copy_(w.to(p.dtype).reshape(p.shape))
            loaded.add(name)
        return loaded


def _map_vae_name(name: str):
    """diffusers name -> this module's name (None for temporal-only parameters)."""
    if "time_conv" in name:
        return None
    n = name
    n = n.replace("mid_block.resnets.0.", "mid.0.").replace("mid_block.attentions.0.", "mid.1.")
    n = n.replace("mid_block.resnets.1.", "mid.2.")
    n = n.replace(".conv_shortcut.", ".shortcut.")
    n = n.replace(".resample.1.", ".conv.")
    import re
    n = re.sub(r"up_blocks\.(\d+)\.resnets\.(\d+)\.", r"up_blocks.\1.\2.", n)
    m = re.match(r"(decoder\.up_blocks\.(\d+))\.upsamplers\.0\.(.*)", n)
    if m:
        n = f"{m.group(1)}.3.{m.group(3)}"
    return n
