"""Deep-compression 3-D autoencoder of HunyuanImage-3
(vllm_omni/diffusion/models/hunyuan_image_3/autoencoder.py:113-383): 32 latent channels at 1/16 of
the image side, 3x3x3 convolutions throughout, and re-sampling by channel<->space shuffles with a
parameter-free shortcut:

  down:  conv to C_out/f channels, fold every (r1, 2, 2) block of positions into channels, and add
         the input folded the same way and averaged over groups of f*C_in/C_out channels;
  up:    conv to C_out*f channels, unfold channels into (r1, 2, 2) blocks of positions, and add the
         input with every channel repeated f*C_out/C_in times, unfolded the same way.

An image is a clip of one latent frame: the encoder sees the picture repeated ``ffactor_temporal``
times, the decoder's temporal up-sampling makes ``ffactor_temporal`` frames of which the last is
the picture (autoencoder.py:592-668).  Parameter names follow the checkpoint
(``decoder.up.{i}.block.{j}.conv1.weight`` ...).  The convolutions are library calls (cuDNN) in
channels-last-3d; the decoder is a few percent of a request next to the 32-layer MoE denoiser.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F
from torch import nn

from ....ops.conv import wide_head_attention


@dataclass
class Conv3dVAEConfig:
    in_channels: int = 3
    out_channels: int = 3
    latent_channels: int = 32
    block_out_channels: tuple = (128, 256, 512, 1024, 1024)
    layers_per_block: int = 2
    ffactor_spatial: int = 16
    ffactor_temporal: int = 4
    scaling_factor: float | None = 0.562679178327931
    shift_factor: float | None = None
    downsample_match_channel: bool = True
    upsample_match_channel: bool = True
    norm_num_groups: int = 32

    @classmethod
    def from_dict(cls, d: dict | None) -> "Conv3dVAEConfig":
        d = d or {}
        known = {k: d[k] for k in cls.__dataclass_fields__ if k in d}
        if "block_out_channels" in known:
            known["block_out_channels"] = tuple(known["block_out_channels"])
        return cls(**known)


def _fold(x: torch.Tensor, r1: int) -> torch.Tensor:
    """[B, C, F*r1, H*2, W*2] -> [B, r1*4*C, F, H, W], channel index (r1, r2, r3, c)."""
    B, C, Fr, Hr, Wr = x.shape
    x = x.view(B, C, Fr // r1, r1, Hr // 2, 2, Wr // 2, 2)
    return x.permute(0, 3, 5, 7, 1, 2, 4, 6).reshape(B, r1 * 4 * C, Fr // r1, Hr // 2, Wr // 2)


def _unfold(x: torch.Tensor, r1: int) -> torch.Tensor:
    """[B, r1*4*C, F, H, W] -> [B, C, F*r1, H*2, W*2]."""
    B, CC, Fr, H, W = x.shape
    C = CC // (r1 * 4)
    x = x.view(B, r1, 2, 2, C, Fr, H, W)
    return x.permute(0, 4, 5, 1, 6, 2, 7, 3).reshape(B, C, Fr * r1, H * 2, W * 2)


class ResnetBlock3d(nn.Module):
    def __init__(self, cin: int, cout: int, g: int = 32):
        super().__init__()
        self.norm1 = nn.GroupNorm(g, cin, eps=1e-6)
        self.conv1 = nn.Conv3d(cin, cout, 3, padding=1)
        self.norm2 = nn.GroupNorm(g, cout, eps=1e-6)
        self.conv2 = nn.Conv3d(cout, cout, 3, padding=1)
        self.nin_shortcut = nn.Conv3d(cin, cout, 1) if cin != cout else None

    def forward(self, x):
        h = self.conv1(F.silu(self.norm1(x)))
        h = self.conv2(F.silu(self.norm2(h)))
        return (x if self.nin_shortcut is None else self.nin_shortcut(x)) + h


class AttnBlock3d(nn.Module):
    """Single-head attention over all positions of the coarsest grid."""

    def __init__(self, c: int, g: int = 32):
        super().__init__()
        self.norm = nn.GroupNorm(g, c, eps=1e-6)
        self.q, self.k, self.v, self.proj_out = (nn.Conv3d(c, c, 1) for _ in range(4))

    def forward(self, x):
        B, C, Fr, H, W = x.shape
        h = self.norm(x)
        q, k, v = (m(h).flatten(2).transpose(1, 2).contiguous() for m in (self.q, self.k, self.v))   # [B, L, C]
        o = wide_head_attention(q, k, v).transpose(1, 2).reshape(B, C, Fr, H, W)
        return x + self.proj_out(o)


class DownsampleFold(nn.Module):
    def __init__(self, cin: int, cout: int, temporal: bool):
        super().__init__()
        self.r1 = 2 if temporal else 1
        f = self.r1 * 4
        self.conv = nn.Conv3d(cin, cout // f, 3, padding=1)
        self.group = f * cin // cout

    def forward(self, x):
        h = _fold(self.conv(x), self.r1)
        s = _fold(x, self.r1)
        B, _, Fr, H, W = s.shape
        return h + s.view(B, h.shape[1], self.group, Fr, H, W).mean(dim=2)


class UpsampleUnfold(nn.Module):
    def __init__(self, cin: int, cout: int, temporal: bool):
        super().__init__()
        self.r1 = 2 if temporal else 1
        f = self.r1 * 4
        self.conv = nn.Conv3d(cin, cout * f, 3, padding=1)
        self.repeats = f * cout // cin

    def forward(self, x):
        return _unfold(self.conv(x), self.r1) + _unfold(x.repeat_interleave(self.repeats, dim=1), self.r1)


class _Level(nn.Module):
    pass


class Encoder3d(nn.Module):
    def __init__(self, c: Conv3dVAEConfig):
        super().__init__()
        ch = c.block_out_channels
        g = c.norm_num_groups
        self.z = c.latent_channels
        self.conv_in = nn.Conv3d(c.in_channels, ch[0], 3, padding=1)
        self.down = nn.ModuleList()
        cin = ch[0]
        ls, lt = math.log2(c.ffactor_spatial), math.log2(c.ffactor_spatial // c.ffactor_temporal)
        for i, cout in enumerate(ch):
            lvl = _Level()
            lvl.block = nn.ModuleList()
            for _ in range(c.layers_per_block):
                lvl.block.append(ResnetBlock3d(cin, cout, g))
                cin = cout
            if i < ls:
                nxt = ch[i + 1] if c.downsample_match_channel else cin
                lvl.downsample = DownsampleFold(cin, nxt, temporal=i >= lt)
                cin = nxt
            self.down.append(lvl)
        self.mid = _Level()
        self.mid.block_1, self.mid.attn_1, self.mid.block_2 = ResnetBlock3d(cin, cin, g), AttnBlock3d(cin, g), ResnetBlock3d(cin, cin, g)
        self.norm_out = nn.GroupNorm(g, cin, eps=1e-6)
        self.conv_out = nn.Conv3d(cin, 2 * self.z, 3, padding=1)
        self.group = cin // (2 * self.z)

    def forward(self, x):
        h = self.conv_in(x)
        for lvl in self.down:
            for b in lvl.block:
                h = b(h)
            if hasattr(lvl, "downsample"):
                h = lvl.downsample(h)
        h = self.mid.block_2(self.mid.attn_1(self.mid.block_1(h)))
        B, C, Fr, H, W = h.shape
        short = h.view(B, C // self.group, self.group, Fr, H, W).mean(dim=2)
        return self.conv_out(F.silu(self.norm_out(h))) + short


class Decoder3d(nn.Module):
    def __init__(self, c: Conv3dVAEConfig):
        super().__init__()
        ch = tuple(reversed(c.block_out_channels))
        g = c.norm_num_groups
        self.z = c.latent_channels
        cin = ch[0]
        self.repeats = cin // self.z
        self.conv_in = nn.Conv3d(self.z, cin, 3, padding=1)
        self.mid = _Level()
        self.mid.block_1, self.mid.attn_1, self.mid.block_2 = ResnetBlock3d(cin, cin, g), AttnBlock3d(cin, g), ResnetBlock3d(cin, cin, g)
        self.up = nn.ModuleList()
        ls, lt = math.log2(c.ffactor_spatial), math.log2(c.ffactor_temporal)
        for i, cout in enumerate(ch):
            lvl = _Level()
            lvl.block = nn.ModuleList()
            for _ in range(c.layers_per_block + 1):
                lvl.block.append(ResnetBlock3d(cin, cout, g))
                cin = cout
            if i < ls or i < lt:
                nxt = ch[i + 1] if c.upsample_match_channel else cin
                lvl.upsample = UpsampleUnfold(cin, nxt, temporal=i < lt)
                cin = nxt
            self.up.append(lvl)
        self.norm_out = nn.GroupNorm(g, cin, eps=1e-6)
        self.conv_out = nn.Conv3d(cin, c.out_channels, 3, padding=1)

    def forward(self, z):
        h = self.conv_in(z) + z.repeat_interleave(self.repeats, dim=1)
        h = self.mid.block_2(self.mid.attn_1(self.mid.block_1(h)))
        for lvl in self.up:
            for b in lvl.block:
                h = b(h)
            if hasattr(lvl, "upsample"):
                h = lvl.upsample(h)
        return self.conv_out(F.silu(self.norm_out(h)))


class AutoencoderKLConv3D(nn.Module):
    def __init__(self, cfg: Conv3dVAEConfig | dict | None = None, with_encoder: bool = False):
        super().__init__()
        self.cfg = cfg if isinstance(cfg, Conv3dVAEConfig) else Conv3dVAEConfig.from_dict(cfg)
        self.encoder = Encoder3d(self.cfg) if with_encoder else None
        self.decoder = Decoder3d(self.cfg)
        self.use_tiling = False
        self.tile_latent = 64                # latent tile side when tiling (64 -> 1024 px)
        self.tile_overlap = 0.25
        self.latent_channels = self.cfg.latent_channels
        self.scale_factor = self.cfg.ffactor_spatial

    def _cl(self, x):
        return x.contiguous(memory_format=torch.channels_last_3d) if x.is_cuda else x

    @torch.no_grad()
    def encode(self, x: torch.Tensor, generator=None, sample: bool = True) -> torch.Tensor:
        """x [B, 3, H, W] in [-1, 1] -> scaled latents [B, z, H/16, W/16]."""
        assert self.encoder is not None, "this autoencoder was built without its encoder"
        x = x[:, :, None].expand(-1, -1, self.cfg.ffactor_temporal, -1, -1)
        mom = self.encoder(self._cl(x.to(self.decoder.conv_in.weight.dtype)))
        mean, logvar = mom.float().chunk(2, dim=1)
        z = mean
        if sample:
            std = torch.exp(0.5 * logvar.clamp(-30.0, 20.0))
            z = mean + std * torch.randn(mean.shape, generator=generator, device=mean.device)
        z = z[:, :, 0]
        if self.cfg.shift_factor:
            z = z - self.cfg.shift_factor
        return z * (self.cfg.scaling_factor or 1.0)

    def _decode_tile(self, z):
        return self.decoder(self._cl(z[:, :, None]))[:, :, -1]

    @torch.no_grad()
    def decode(self, z: torch.Tensor) -> torch.Tensor:
        """Scaled latents [B, z, h, w] -> image [B, 3, 16h, 16w]."""
        z = z.to(self.decoder.conv_in.weight.dtype) / (self.cfg.scaling_factor or 1.0)
        if self.cfg.shift_factor:
            z = z + self.cfg.shift_factor
        t = self.tile_latent
        if not self.use_tiling or (z.shape[-1] <= t and z.shape[-2] <= t):
            return self._decode_tile(z)
        # overlapping tiles, blended linearly over the overlap (autoencoder.py:536-563)
        s = self.cfg.ffactor_spatial
        step = int(t * (1 - self.tile_overlap))
        blend = int(t * s * self.tile_overlap)
        keep = step * s
        rows = []
        for i in range(0, z.shape[-2], step):
            rows.append([self._decode_tile(z[..., i:i + t, j:j + t]) for j in range(0, z.shape[-1], step)])
        out_rows = []
        for ri, row in enumerate(rows):
            out = []
            for ci, tile in enumerate(row):
                tile = tile.clone()
                if ri > 0:
                    up = rows[ri - 1][ci]
                    n = min(blend, up.shape[-2], tile.shape[-2])
                    wgt = (torch.arange(n, device=tile.device, dtype=tile.dtype) / n).view(1, 1, n, 1)
                    tile[..., :n, :] = up[..., -n:, :][..., :, :tile.shape[-1]] * (1 - wgt) + tile[..., :n, :] * wgt
                if ci > 0:
                    left = row[ci - 1]
                    n = min(blend, left.shape[-1], tile.shape[-1])
                    wgt = (torch.arange(n, device=tile.device, dtype=tile.dtype) / n).view(1, 1, 1, n)
                    tile[..., :, :n] = left[..., :tile.shape[-2], -n:] * (1 - wgt) + tile[..., :, :n] * wgt
                row[ci] = tile
                out.append(tile[..., :keep, :keep])
            out_rows.append(torch.cat(out, dim=-1))
        return torch.cat(out_rows, dim=-2)[..., :z.shape[-2] * s, :z.shape[-1] * s]

    def load_weights(self, weights) -> set:
        params = dict(self.named_parameters())
        loaded = set()
        for n, w in weights:
            p = params.get(n)
            if p is None or p.shape != w.shape:
                continue
            p.data.copy_(w.to(p.dtype))
            loaded.add(n)
        return loaded
