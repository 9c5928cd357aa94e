"""The 2-D KL autoencoder of the FLUX / SD3 / Z-Image / LongCat / Ovis checkpoints (diffusers
``AutoencoderKL``; the reference imports it from diffusers and wraps it for patch-parallel decoding,
vllm_omni/diffusion/distributed/vae_patch_parallel.py:463).

Decoder: conv_in -> mid block (ResNet, single-head attention over pixels, ResNet) -> one up block
per entry of ``block_out_channels`` (``layers_per_block + 1`` ResNets, nearest 2x up-sampling + 3x3
conv except in the last) -> GroupNorm(32) -> SiLU -> conv_out.  The encoder mirrors it and ends in
mean / log-variance channels.  Latents are ``z / scaling_factor + shift_factor`` before decoding.
The module tree and parameter names equal the diffusers checkpoint (``decoder.up_blocks.0.resnets.1.
conv1.weight`` ...), so ``load_weights`` is a plain name match; the older attention names
(``query/key/value/proj_attn``) are accepted too.

Convolutions and group norms run in channels_last through PyTorch (cuDNN); the tiled decode bounds
the activation memory of large images and is what the patch-parallel wrapper distributes.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ....ops.conv import wide_head_attention


@dataclass
class AutoencoderKLConfig:
    in_channels: int = 3
    out_channels: int = 3
    latent_channels: int = 16
    block_out_channels: tuple = (128, 256, 512, 512)
    layers_per_block: int = 2
    norm_num_groups: int = 32
    scaling_factor: float = 0.3611
    shift_factor: float | None = 0.1159
    use_quant_conv: bool = False
    use_post_quant_conv: bool = False
    mid_block_add_attention: bool = True

    @property
    def spatial_scale(self) -> int:
        return 2 ** (len(self.block_out_channels) - 1)

    @classmethod
    def from_dict(cls, d):
        keys = set(cls.__dataclass_fields__)
        return cls(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in d.items() if k in keys})


class ResnetBlock2D(nn.Module):
    def __init__(self, cin, cout, groups):
        super().__init__()
        self.norm1 = nn.GroupNorm(groups, cin, eps=1e-6)
        self.conv1 = nn.Conv2d(cin, cout, 3, padding=1)
        self.norm2 = nn.GroupNorm(groups, cout, eps=1e-6)
        self.conv2 = nn.Conv2d(cout, cout, 3, padding=1)
        self.conv_shortcut = nn.Conv2d(cin, cout, 1) if cin != cout else None

    def forward(self, x):
        h = self.conv1(F.silu(self.norm1(x)))
        h = self.conv2(F.silu(self.norm2(h)))
        return h + (x if self.conv_shortcut is None else self.conv_shortcut(x))


class PixelAttention(nn.Module):
    """Single-head self-attention over the H*W pixels of the mid block."""

    def __init__(self, ch, groups):
        super().__init__()
        self.group_norm = nn.GroupNorm(groups, ch, eps=1e-6)
        self.to_q, self.to_k, self.to_v = nn.Linear(ch, ch), nn.Linear(ch, ch), nn.Linear(ch, ch)
        self.to_out = nn.ModuleList([nn.Linear(ch, ch)])

    def forward(self, x):
        B, C, H, W = x.shape
        h = self.group_norm(x).reshape(B, C, H * W).transpose(1, 2)
        o = wide_head_attention(self.to_q(h), self.to_k(h), self.to_v(h))       # GEMM / softmax / GEMM kernels on a GPU in bf16
        return x + self.to_out[0](o).transpose(1, 2).reshape(B, C, H, W)


class MidBlock(nn.Module):
    def __init__(self, ch, groups, attention=True):
        super().__init__()
        self.resnets = nn.ModuleList([ResnetBlock2D(ch, ch, groups), ResnetBlock2D(ch, ch, groups)])
        self.attentions = nn.ModuleList([PixelAttention(ch, groups)] if attention else [])

    def forward(self, x):
        x = self.resnets[0](x)
        for a in self.attentions:
            x = a(x)
        return self.resnets[1](x)


class _Resample(nn.Module):
    def __init__(self, ch, down):
        super().__init__()
        self.down = down
        self.conv = nn.Conv2d(ch, ch, 3, stride=2 if down else 1, padding=0 if down else 1)

    def forward(self, x):
        if self.down:
            return self.conv(F.pad(x, (0, 1, 0, 1)))          # asymmetric padding of the strided conv
        return self.conv(F.interpolate(x, scale_factor=2.0, mode="nearest"))


class UpBlock(nn.Module):
    def __init__(self, cin, cout, n, groups, upsample):
        super().__init__()
        self.resnets = nn.ModuleList([ResnetBlock2D(cin if i == 0 else cout, cout, groups) for i in range(n)])
        self.upsamplers = nn.ModuleList([_Resample(cout, False)]) if upsample else None

    def forward(self, x):
        for r in self.resnets:
            x = r(x)
        return self.upsamplers[0](x) if self.upsamplers is not None else x


class DownBlock(nn.Module):
    def __init__(self, cin, cout, n, groups, downsample):
        super().__init__()
        self.resnets = nn.ModuleList([ResnetBlock2D(cin if i == 0 else cout, cout, groups) for i in range(n)])
        self.downsamplers = nn.ModuleList([_Resample(cout, True)]) if downsample else None

    def forward(self, x):
        for r in self.resnets:
            x = r(x)
        return self.downsamplers[0](x) if self.downsamplers is not None else x


class Decoder(nn.Module):
    def __init__(self, c: AutoencoderKLConfig):
        super().__init__()
        ch = list(c.block_out_channels)
        g = c.norm_num_groups
        self.conv_in = nn.Conv2d(c.latent_channels, ch[-1], 3, padding=1)
        self.mid_block = MidBlock(ch[-1], g, c.mid_block_add_attention)
        rev = ch[::-1]
        blocks, prev = [], rev[0]
        for i, co in enumerate(rev):
            blocks.append(UpBlock(prev, co, c.layers_per_block + 1, g, upsample=i < len(rev) - 1))
            prev = co
        self.up_blocks = nn.ModuleList(blocks)
        self.conv_norm_out = nn.GroupNorm(g, ch[0], eps=1e-6)
        self.conv_out = nn.Conv2d(ch[0], c.out_channels, 3, padding=1)

    def forward(self, z):
        x = self.mid_block(self.conv_in(z))
        for b in self.up_blocks:
            x = b(x)
        return self.conv_out(F.silu(self.conv_norm_out(x)))


class Encoder(nn.Module):
    def __init__(self, c: AutoencoderKLConfig):
        super().__init__()
        ch = list(c.block_out_channels)
        g = c.norm_num_groups
        self.conv_in = nn.Conv2d(c.in_channels, ch[0], 3, padding=1)
        blocks, prev = [], ch[0]
        for i, co in enumerate(ch):
            blocks.append(DownBlock(prev, co, c.layers_per_block, g, downsample=i < len(ch) - 1))
            prev = co
        self.down_blocks = nn.ModuleList(blocks)
        self.mid_block = MidBlock(ch[-1], g, c.mid_block_add_attention)
        self.conv_norm_out = nn.GroupNorm(g, ch[-1], eps=1e-6)
        self.conv_out = nn.Conv2d(ch[-1], 2 * c.latent_channels, 3, padding=1)

    def forward(self, x):
        x = self.conv_in(x)
        for b in self.down_blocks:
            x = b(x)
        return self.conv_out(F.silu(self.conv_norm_out(self.mid_block(x))))


_OLD_ATTN = {"query": "to_q", "key": "to_k", "value": "to_v", "proj_attn": "to_out.0"}
_BFL_ATTN = {"q": "to_q", "k": "to_k", "v": "to_v", "proj_out": "to_out.0", "norm": "group_norm"}


def bfl_to_diffusers_name(name: str, num_blocks: int) -> str:
    """Names of the original FLUX autoencoder file (``ae.safetensors``, also what BAGEL ships:
    ``decoder.up.3.block.0.norm1``, ``decoder.mid.attn_1.q``, ``encoder.down.0.downsample.conv``) -> the
    diffusers names this module uses.  The original numbers its up stages from the output side."""
    p = name.split(".")
    if len(p) < 3 or p[0] not in ("encoder", "decoder"):
        return name
    side, rest = p[0], p[1:]
    if rest[0] == "norm_out":
        return ".".join([side, "conv_norm_out"] + rest[1:])
    if rest[0] == "mid":
        if rest[1] in ("block_1", "block_2"):
            tail = ["conv_shortcut" if t == "nin_shortcut" else t for t in rest[2:]]
            return ".".join([side, "mid_block", "resnets", "0" if rest[1] == "block_1" else "1"] + tail)
        if rest[1] == "attn_1":
            return ".".join([side, "mid_block", "attentions", "0", _BFL_ATTN.get(rest[2], rest[2])] + rest[3:])
    if rest[0] in ("up", "down") and len(rest) > 3:
        i = int(rest[1])
        blk = ("up_blocks", str(num_blocks - 1 - i)) if rest[0] == "up" else ("down_blocks", str(i))
        if rest[2] == "block":
            tail = ["conv_shortcut" if t == "nin_shortcut" else t for t in rest[4:]]
            return ".".join([side, *blk, "resnets", rest[3]] + tail)
        if rest[2] in ("upsample", "downsample"):
            return ".".join([side, *blk, "upsamplers" if rest[2] == "upsample" else "downsamplers", "0"] + rest[3:])
    return name


class AutoencoderKL(nn.Module):
    def __init__(self, cfg: AutoencoderKLConfig | None = None, with_encoder: bool = False):
        super().__init__()
        self.cfg = c = cfg or AutoencoderKLConfig()
        self.decoder = Decoder(c)
        self.encoder = Encoder(c) if with_encoder else None
        self.post_quant_conv = nn.Conv2d(c.latent_channels, c.latent_channels, 1) if c.use_post_quant_conv else None
        self.quant_conv = nn.Conv2d(2 * c.latent_channels, 2 * c.latent_channels, 1) if (c.use_quant_conv and with_encoder) else None
        self.use_tiling = False
        self.tile_latent, self.tile_overlap = 64, 16
        self.decoder_impl = os.environ.get("OMNI_VAE_IMPL", "nhwc")      # "nhwc" (own kernels) | "torch" (cuDNN)
        self._nhwc = None
        for p in self.parameters():
            p.requires_grad_(False)

    @property
    def dtype(self):
        return self.decoder.conv_in.weight.dtype

    # ---- latents <-> model space
    def denormalize(self, z):
        z = z / self.cfg.scaling_factor
        return z + self.cfg.shift_factor if self.cfg.shift_factor else z

    def normalize(self, z):
        z = z - self.cfg.shift_factor if self.cfg.shift_factor else z
        return z * self.cfg.scaling_factor

    @torch.no_grad()
    def decode(self, z: torch.Tensor, denormalize: bool = True) -> torch.Tensor:
        """z: [B, C, h, w] (or [B, C, 1, h, w]) scheduler-space latents -> images [B, 3, 8h, 8w] in [-1, 1]."""
        if z.dim() == 5:
            z = z[:, :, 0]
        z = z.to(self.dtype)
        if denormalize:
            z = self.denormalize(z)
        tiled = self.use_tiling and max(z.shape[-2:]) > self.tile_latent
        if z.is_cuda and self.dtype == torch.bfloat16 and not tiled and self.decoder_impl != "torch":
            # channels-last decode on the implicit-GEMM / GroupNorm kernels of this library
            if self._nhwc is None:
                from .nhwc_decoder_kl import NHWCDecoderKL
                self._nhwc = NHWCDecoderKL(self.decoder, self.post_quant_conv, torch.bfloat16) \
                    if NHWCDecoderKL.supported(self.decoder) else False
            if self._nhwc:
                return self._nhwc(z.contiguous()).to(self.dtype)
        if self.post_quant_conv is not None:
            z = self.post_quant_conv(z)
        z = z.contiguous(memory_format=torch.channels_last)
        if self.use_tiling and max(z.shape[-2:]) > self.tile_latent:
            return self._tiled_decode(z)
        return self.decoder(z).clamp(-1, 1)

    def _tiled_decode(self, z):
        """Overlapping latent tiles, linear cross-fade over the overlap in pixel space."""
        T, O, s = self.tile_latent, self.tile_overlap, self.cfg.spatial_scale
        B, _, h, w = z.shape
        out = z.new_zeros(B, self.cfg.out_channels, h * s, w * s, dtype=torch.float32)
        wsum = z.new_zeros(1, 1, h * s, w * s, dtype=torch.float32)
        step = T - O
        for y0 in range(0, max(1, h - O), step):
            for x0 in range(0, max(1, w - O), step):
                y1, x1 = min(h, y0 + T), min(w, x0 + T)
                tile = self.decoder(z[:, :, y0:y1, x0:x1]).float()
                wy, wx = _ramp(y1 - y0, O, y0 > 0, y1 < h, s, z.device), _ramp(x1 - x0, O, x0 > 0, x1 < w, s, z.device)
                m = wy[:, None] * wx[None, :]
                out[:, :, y0 * s:y1 * s, x0 * s:x1 * s] += tile * m
                wsum[:, :, y0 * s:y1 * s, x0 * s:x1 * s] += m
        return (out / wsum).clamp(-1, 1).to(z.dtype)

    @torch.no_grad()
    def encode(self, x: torch.Tensor, sample: bool = False, generator=None) -> torch.Tensor:
        """images [B, 3, H, W] in [-1, 1] -> scheduler-space latents (mode of the posterior unless ``sample``)."""
        if self.encoder is None:
            raise RuntimeError("this AutoencoderKL was built without its encoder")
        m = self.encoder(x.to(self.dtype).contiguous(memory_format=torch.channels_last))
        if self.quant_conv is not None:
            m = self.quant_conv(m)
        mean, logvar = m.chunk(2, dim=1)
        if sample:
            std = torch.exp(0.5 * logvar.float().clamp(-30, 20))
            mean = mean.float() + std * torch.randn(mean.shape, generator=generator, device=mean.device)
        return self.normalize(mean.float())

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        own = dict(self.named_parameters())
        loaded = set()
        for name, w in weights:
            n = name
            for old, new in _OLD_ATTN.items():
                n = n.replace(f".attentions.0.{old}.", f".attentions.0.{new}.")
            if n not in own:
                n = bfl_to_diffusers_name(name, len(self.cfg.block_out_channels))
            if n not in own:
                continue
            p = own[n]
            p.copy_(w.to(p.dtype).reshape(p.shape))          # old checkpoints store the attention linears as 1x1 convs
            loaded.add(name)
        return loaded


def _ramp(n, overlap, fade_in, fade_out, scale, device):
    """Per-pixel blending weight along one axis of a tile of ``n`` latent rows."""
    w = torch.ones(n * scale, device=device)
    k = min(overlap, n) * scale
    r = (torch.arange(k, device=device).float() + 0.5) / k
    if fade_in:
        w[:k] = r
    if fade_out:
        w[-k:] = torch.minimum(w[-k:], r.flip(0))
    return w
