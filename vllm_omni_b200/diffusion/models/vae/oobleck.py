"""Oobleck audio autoencoder of Stable Audio Open (diffusers' ``AutoencoderOobleck``, which the
reference loads from the checkpoint's ``vae/`` folder: vllm_omni/diffusion/models/stable_audio/
pipeline_stable_audio.py): latents [B, 64, L] at 44.1 kHz / 2048 <-> stereo waveform [B, 2, 2048 L].

Decoder: conv(7) to ``channels * multiples[-1]``; per stage a Snake activation, a transposed conv of
kernel ``2 stride`` / padding ``ceil(stride / 2)`` that halves the width, and three residual units
(Snake, dilated conv(7) with dilation 1 / 3 / 9, Snake, conv(1)); a last Snake and a bias-free conv(7)
to the audio channels.  The encoder mirrors it (residual units, Snake, strided conv of kernel
``2 stride``) and ends in a conv(3) to mean and scale of the latent.  Snake is
``x + sin^2(e^alpha x) / (e^beta + 1e-9)`` with one alpha and beta per channel.

Every convolution of the checkpoint is weight-normalised (``weight_g`` / ``weight_v``, or the
``parametrizations.weight.original0/1`` names of newer torch); the norm is folded into a plain weight
when the tensors are loaded.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
from torch import nn


@dataclass
class OobleckConfig:
    encoder_hidden_size: int = 128
    downsampling_ratios: tuple = (2, 4, 4, 8, 8)
    channel_multiples: tuple = (1, 2, 4, 8, 16)
    decoder_channels: int = 128
    decoder_input_channels: int = 64
    audio_channels: int = 2
    sampling_rate: int = 44100

    @classmethod
    def from_dict(cls, d: dict) -> "OobleckConfig":
        keys = set(cls.__dataclass_fields__)
        return cls(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in d.items() if k in keys})

    @property
    def hop_length(self) -> int:
        return int(math.prod(self.downsampling_ratios))


class Snake1d(nn.Module):
    def __init__(self, ch, **kw):
        super().__init__()
        self.alpha = nn.Parameter(torch.zeros(1, ch, 1, **kw), requires_grad=False)
        self.beta = nn.Parameter(torch.zeros(1, ch, 1, **kw), requires_grad=False)

    def forward(self, x):
        xf = x.float()
        a, b = self.alpha.float().exp(), self.beta.float().exp()
        return (xf + (b + 1e-9).reciprocal() * torch.sin(a * xf).pow(2)).to(x.dtype)


class ResidualUnit(nn.Module):
    def __init__(self, ch, dilation, **kw):
        super().__init__()
        self.snake1 = Snake1d(ch, **kw)
        self.conv1 = nn.Conv1d(ch, ch, 7, dilation=dilation, padding=3 * dilation, **kw)
        self.snake2 = Snake1d(ch, **kw)
        self.conv2 = nn.Conv1d(ch, ch, 1, **kw)

    def forward(self, x):
        return x + self.conv2(self.snake2(self.conv1(self.snake1(x))))


class DecoderBlock(nn.Module):
    def __init__(self, cin, cout, stride, **kw):
        super().__init__()
        self.snake1 = Snake1d(cin, **kw)
        self.conv_t1 = nn.ConvTranspose1d(cin, cout, 2 * stride, stride=stride, padding=math.ceil(stride / 2), **kw)
        self.res_unit1, self.res_unit2, self.res_unit3 = (ResidualUnit(cout, d, **kw) for d in (1, 3, 9))

    def forward(self, x):
        return self.res_unit3(self.res_unit2(self.res_unit1(self.conv_t1(self.snake1(x)))))


class EncoderBlock(nn.Module):
    def __init__(self, cin, cout, stride, **kw):
        super().__init__()
        self.res_unit1, self.res_unit2, self.res_unit3 = (ResidualUnit(cin, d, **kw) for d in (1, 3, 9))
        self.snake1 = Snake1d(cin, **kw)
        self.conv1 = nn.Conv1d(cin, cout, 2 * stride, stride=stride, padding=math.ceil(stride / 2), **kw)

    def forward(self, x):
        return self.conv1(self.snake1(self.res_unit3(self.res_unit2(self.res_unit1(x)))))


class OobleckDecoder(nn.Module):
    def __init__(self, c: OobleckConfig, **kw):
        super().__init__()
        mult = (1,) + tuple(c.channel_multiples)
        strides = tuple(c.downsampling_ratios)[::-1]
        ch = c.decoder_channels
        self.conv1 = nn.Conv1d(c.decoder_input_channels, ch * mult[-1], 7, padding=3, **kw)
        n = len(strides)
        self.block = nn.ModuleList([DecoderBlock(ch * mult[n - i], ch * mult[n - i - 1], s, **kw) for i, s in enumerate(strides)])
        self.snake1 = Snake1d(ch, **kw)
        self.conv2 = nn.Conv1d(ch, c.audio_channels, 7, padding=3, bias=False, **kw)

    def forward(self, z):
        x = self.conv1(z)
        for b in self.block:
            x = b(x)
        return self.conv2(self.snake1(x))


class OobleckEncoder(nn.Module):
    def __init__(self, c: OobleckConfig, **kw):
        super().__init__()
        mult = (1,) + tuple(c.channel_multiples)
        ch = c.encoder_hidden_size
        self.conv1 = nn.Conv1d(c.audio_channels, ch, 7, padding=3, **kw)
        self.block = nn.ModuleList([EncoderBlock(ch * mult[i], ch * mult[i + 1], s, **kw)
                                    for i, s in enumerate(c.downsampling_ratios)])
        self.snake1 = Snake1d(ch * mult[-1], **kw)
        self.conv2 = nn.Conv1d(ch * mult[-1], c.encoder_hidden_size, 3, padding=1, **kw)      # mean | scale

    def forward(self, wav):
        x = self.conv1(wav)
        for b in self.block:
            x = b(x)
        return self.conv2(self.snake1(x))


class AutoencoderOobleck(nn.Module):
    def __init__(self, cfg: OobleckConfig | None = None, dtype=torch.float32, device=None, with_encoder: bool = False):
        super().__init__()
        self.config = c = cfg or OobleckConfig()
        kw = dict(dtype=dtype, device=device)
        self.decoder = OobleckDecoder(c, **kw)
        self.encoder = OobleckEncoder(c, **kw) if with_encoder else None
        for p in self.parameters():
            p.requires_grad_(False)

    @property
    def hop_length(self) -> int:
        return self.config.hop_length

    @torch.no_grad()
    def decode(self, z: torch.Tensor) -> torch.Tensor:
        return self.decoder(z.to(self.decoder.conv1.weight.dtype))

    @torch.no_grad()
    def encode(self, wav: torch.Tensor, generator=None, sample: bool = True) -> torch.Tensor:
        """Waveform [B, 2, T] -> latent [B, 64, T / hop]: mean + softplus(scale) * noise (or the mean)."""
        if self.encoder is None:
            raise ValueError("this autoencoder was built without its encoder")
        mean, scale = self.encoder(wav.to(self.decoder.conv1.weight.dtype)).chunk(2, dim=1)
        if not sample:
            return mean
        std = torch.nn.functional.softplus(scale) + 1e-4
        return mean + std * torch.randn(mean.shape, generator=generator, device=mean.device, dtype=mean.dtype)

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        """diffusers names under ``decoder.`` / ``encoder.``; weight-norm pairs are folded as they complete."""
        params = dict(self.named_parameters())
        pending: dict[str, dict] = {}
        loaded = set()
        alias = {"parametrizations.weight.original0": "weight_g", "parametrizations.weight.original1": "weight_v"}
        for n, w in weights:
            for a, b in alias.items():
                if n.endswith(a):
                    n_key, kind = n[:-len(a)] + "weight", b
                    break
            else:
                if n.endswith(("weight_g", "weight_v")):
                    n_key, kind = n[:-2], n[-8:]
                else:
                    n_key, kind = n, None
            if n_key not in params:
                continue
            if kind is None:
                params[n_key].copy_(w.to(params[n_key].dtype).reshape(params[n_key].shape))
                loaded.add(n)
                continue
            slot = pending.setdefault(n_key, {})
            slot[kind] = (n, w.float())
            if len(slot) == 2:
                (ng, g), (nv, v) = slot["weight_g"], slot["weight_v"]
                norm = v.flatten(1).norm(dim=1).view(-1, *([1] * (v.dim() - 1)))
                params[n_key].copy_((v * (g / norm)).to(params[n_key].dtype))
                loaded.update((ng, nv))
                del pending[n_key]
        return loaded
