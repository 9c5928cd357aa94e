"""Stable Audio DiT (vllm_omni/diffusion/models/stable_audio/stable_audio_transformer.py:60-602) and
the small projection model that turns text states and the start / end seconds into its conditioning
(diffusers' ``StableAudioProjectionModel``, loaded by the reference's pipeline).

Latent [B, C, L]: a residual 1x1 convolution, a projection to the model width, and ONE extra token in
front that carries the global conditioning (projected [start | end] seconds embedding plus the
time embedding: Gaussian Fourier features of the noise level through a two-layer MLP).  Blocks:
LayerNorm -> self-attention whose rotary embedding turns only the first half of every head (the
half-split convention), LayerNorm -> cross-attention to the projected text + seconds tokens with
grouped key / value heads, LayerNorm -> SwiGLU feed-forward (value half first, gate half second).
The extra token is dropped after the output projection and a residual 1x1 convolution closes.

Checkpoint names are diffusers': ``transformer_blocks.N.{norm1,norm2,norm3}``, ``attn1|attn2.to_q/
to_k/to_v/to_out.0``, ``ff.net.0.proj`` / ``ff.net.2``, ``time_proj.weight``, ``timestep_proj.0|2``
(also ``linear_1|2``), ``global_proj.0|2``, ``cross_attention_proj.0|2``, ``preprocess_conv``,
``proj_in``, ``proj_out``, ``postprocess_conv``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ....ops import fused
from ....ops.attention import attention, attention_reference
from ...layers.linear import FusedLinear


@dataclass
class StableAudioDiTConfig:
    sample_size: int = 1024
    in_channels: int = 64
    num_layers: int = 24
    attention_head_dim: int = 64
    num_attention_heads: int = 24
    num_key_value_attention_heads: int = 12
    out_channels: int = 64
    cross_attention_dim: int = 768
    time_proj_dim: int = 256
    global_states_input_dim: int = 1536
    cross_attention_input_dim: int = 768
    ff_mult: int = 4

    @classmethod
    def from_dict(cls, d: dict) -> "StableAudioDiTConfig":
        keys = set(cls.__dataclass_fields__)
        return cls(**{k: v for k, v in d.items() if k in keys})


def rotary_table(rotary_dim: int, length: int, theta: float = 10000.0, device=None):
    """cos / sin [length, rotary_dim]: ``rotary_dim / 2`` frequencies, tiled twice (half-split layout)."""
    inv = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32, device=device)[: rotary_dim // 2] / rotary_dim))
    ang = torch.arange(length, dtype=torch.float32, device=device)[:, None] * inv[None]
    return torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)


def apply_partial_rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B, S, H, Dh]: the first ``cos.shape[-1]`` entries of every head are rotated, the rest pass."""
    r = cos.shape[-1]
    xr = x[..., :r].float()
    a, b = xr[..., : r // 2], xr[..., r // 2:]
    rot = xr * cos[None, :, None, :] + torch.cat([-b, a], -1) * sin[None, :, None, :]
    return torch.cat([rot.to(x.dtype), x[..., r:]], -1)


def _mha(q, k, v):
    if q.is_cuda and q.shape[-1] in (64, 128) and q.dtype == torch.bfloat16:
        return attention(q.contiguous(), k.contiguous(), v.contiguous())
    return attention_reference(q, k, v)


class StableAudioBlock(nn.Module):
    def __init__(self, c: StableAudioDiTConfig, dtype, device):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        D = c.num_attention_heads * c.attention_head_dim
        self.H, self.Hkv, self.Dh = c.num_attention_heads, c.num_key_value_attention_heads, c.attention_head_dim
        self.norm1, self.norm2, self.norm3 = (nn.LayerNorm(D, **kw) for _ in range(3))
        self.qkv = FusedLinear(D, 3 * D, bias=False, **kw)
        self.attn_out = FusedLinear(D, D, bias=False, **kw)
        self.q2 = FusedLinear(D, D, bias=False, **kw)
        self.kv2 = FusedLinear(c.cross_attention_dim, 2 * self.Hkv * self.Dh, bias=False, **kw)
        self.cross_out = FusedLinear(D, D, bias=False, **kw)
        self.ff_in = FusedLinear(D, 2 * c.ff_mult * D, **kw)          # rows: gate half first (swapped at load), value half second
        self.ff_out = FusedLinear(c.ff_mult * D, D, **kw)

    def cross_kv(self, ctx):
        """Keys / values of the conditioning tokens, expanded to the query heads: constant over the steps."""
        B, S, _ = ctx.shape
        kv = self.kv2(ctx).view(B, S, 2, self.Hkv, self.Dh)
        rep = self.H // self.Hkv
        k = kv[:, :, 0].unsqueeze(3).expand(-1, -1, -1, rep, -1).reshape(B, S, self.H, self.Dh)
        v = kv[:, :, 1].unsqueeze(3).expand(-1, -1, -1, rep, -1).reshape(B, S, self.H, self.Dh)
        return k.contiguous(), v.contiguous()

    def forward(self, x, kv, cos, sin):
        B, S, D = x.shape
        H, Dh = self.H, self.Dh
        qkv = self.qkv(self.norm1(x)).view(B, S, 3, H, Dh)
        q, k = apply_partial_rotary(qkv[:, :, 0], cos, sin), apply_partial_rotary(qkv[:, :, 1], cos, sin)
        x = self.attn_out(_mha(q, k, qkv[:, :, 2]).reshape(B, S, D).contiguous(), residual=x)
        q = self.q2(self.norm2(x)).view(B, S, H, Dh)
        x = self.cross_out(_mha(q, kv[0], kv[1]).reshape(B, S, D).contiguous(), residual=x)
        return self.ff_out(fused.silu_mul(self.ff_in(self.norm3(x))), residual=x)


class StableAudioDiTModel(nn.Module):
    def __init__(self, cfg: StableAudioDiTConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = c = cfg
        kw = dict(dtype=dtype, device=device)
        D = c.num_attention_heads * c.attention_head_dim
        self.inner_dim = D
        self.time_freqs = nn.Parameter(torch.randn(c.time_proj_dim // 2, **kw), requires_grad=False)
        self.time1, self.time2 = FusedLinear(c.time_proj_dim, D, **kw), FusedLinear(D, D, **kw)
        self.global1 = FusedLinear(c.global_states_input_dim, D, bias=False, **kw)
        self.global2 = FusedLinear(D, D, bias=False, **kw)
        self.cross1 = FusedLinear(c.cross_attention_input_dim, c.cross_attention_dim, bias=False, **kw)
        self.cross2 = FusedLinear(c.cross_attention_dim, c.cross_attention_dim, bias=False, **kw)
        self.preprocess_conv = FusedLinear(c.in_channels, c.in_channels, bias=False, **kw)       # 1x1 conv over channels
        self.proj_in = FusedLinear(c.in_channels, D, bias=False, **kw)
        self.blocks = nn.ModuleList([StableAudioBlock(c, dtype, device) for _ in range(c.num_layers)])
        self.proj_out = FusedLinear(D, c.out_channels, bias=False, **kw)
        self.postprocess_conv = FusedLinear(c.out_channels, c.out_channels, bias=False, **kw)
        for p in self.parameters():
            p.requires_grad_(False)
        self._rope = None

    def rope(self, length: int, device):
        if self._rope is None or self._rope[0].shape[0] != length or self._rope[0].device != torch.device(device):
            self._rope = rotary_table(self.cfg.attention_head_dim // 2, length, device=device)
        return self._rope

    def conditioning(self, encoder_hidden_states):
        """Projected conditioning tokens and every block's cross-attention keys / values."""
        ctx = self.cross2(self.cross1(encoder_hidden_states.to(self.proj_in.weight.dtype).contiguous(), act="silu"))
        return [blk.cross_kv(ctx) for blk in self.blocks]

    @torch.no_grad()
    def forward(self, hidden_states, timestep, encoder_hidden_states=None, global_hidden_states=None, cross_kv=None):
        """hidden_states [B, C, L], timestep [B] or [1] (atan(sigma) * 2 / pi), encoder_hidden_states
        [B, S, Dc] (or ``cross_kv`` from ``conditioning``), global_hidden_states [B, 1, Dg] -> [B, C, L]."""
        dt = self.proj_in.weight.dtype
        B, C, L = hidden_states.shape
        if cross_kv is None:
            cross_kv = self.conditioning(encoder_hidden_states)
        t = timestep.reshape(-1).float().expand(B) if timestep.numel() == 1 else timestep.reshape(-1).float()
        ang = 2 * math.pi * t[:, None] * self.time_freqs.float()[None]
        temb = self.time2(self.time1(torch.cat([ang.cos(), ang.sin()], -1).to(dt), act="silu"))
        g = self.global2(self.global1(global_hidden_states.to(dt).reshape(B, -1).contiguous(), act="silu")) + temb
        x = hidden_states.to(dt).transpose(1, 2).contiguous()                       # [B, L, C]
        x = self.preprocess_conv(x, residual=x)
        x = torch.cat([g[:, None], self.proj_in(x)], dim=1).contiguous()            # [B, 1 + L, D]
        cos, sin = self.rope(L + 1, x.device)
        for blk, kv in zip(self.blocks, cross_kv):
            x = blk(x, kv, cos, sin)
        y = self.proj_out(x[:, 1:].contiguous())
        y = self.postprocess_conv(y, residual=y)
        return y.transpose(1, 2)

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        c = self.cfg
        D = self.inner_dim
        kvd = c.num_key_value_attention_heads * c.attention_head_dim
        Fi = c.ff_mult * D
        top = {"time_proj.weight": (self.time_freqs, None),
               "timestep_proj.0": self.time1, "timestep_proj.linear_1": self.time1,
               "timestep_proj.2": self.time2, "timestep_proj.linear_2": self.time2,
               "global_proj.0": self.global1, "global_proj.linear_1": self.global1,
               "global_proj.2": self.global2, "global_proj.linear_2": self.global2,
               "cross_attention_proj.0": self.cross1, "cross_attention_proj.2": self.cross2,
               "preprocess_conv": self.preprocess_conv, "postprocess_conv": self.postprocess_conv,
               "proj_in": self.proj_in, "proj_out": self.proj_out}
        loaded = set()
        for n, w in weights:
            tgt, sl = None, None
            stem, _, leaf = n.rpartition(".")
            if n == "time_proj.weight":
                tgt = self.time_freqs
            elif stem in top:
                tgt = getattr(top[stem], leaf, None)
            elif n.startswith("transformer_blocks."):
                p = n.split(".")
                blk, rest = self.blocks[int(p[1])], ".".join(p[2:])
                if p[2] in ("norm1", "norm2", "norm3"):
                    tgt = getattr(getattr(blk, p[2]), leaf)
                elif rest in ("attn1.to_q.weight", "attn1.to_k.weight", "attn1.to_v.weight"):
                    i = ("to_q", "to_k", "to_v").index(p[3])
                    tgt, sl = blk.qkv.weight, (i * D, (i + 1) * D)
                elif rest == "attn1.to_out.0.weight":
                    tgt = blk.attn_out.weight
                elif rest == "attn2.to_q.weight":
                    tgt = blk.q2.weight
                elif rest in ("attn2.to_k.weight", "attn2.to_v.weight"):
                    i = ("to_k", "to_v").index(p[3])
                    tgt, sl = blk.kv2.weight, (i * kvd, (i + 1) * kvd)
                elif rest == "attn2.to_out.0.weight":
                    tgt = blk.cross_out.weight
                elif rest.startswith("ff.net.0.proj."):          # checkpoint rows: value | gate; ours: gate | value
                    dst = getattr(blk.ff_in, leaf)
                    dst[:Fi].copy_(w[Fi:].to(dst.dtype))
                    dst[Fi:].copy_(w[:Fi].to(dst.dtype))
                    loaded.add(n)
                    continue
                elif rest.startswith("ff.net.2."):
                    tgt = getattr(blk.ff_out, leaf)
            if tgt is None:
                continue
            dst = tgt if sl is None else tgt[sl[0]:sl[1]]
            dst.copy_(w.to(dst.dtype).reshape(dst.shape))
            loaded.add(n)
        return loaded


# ----------------------------------------------------------------------------- projection model
@dataclass
class StableAudioProjectionConfig:
    text_encoder_dim: int = 768
    conditioning_dim: int = 768
    min_value: float = 0.0
    max_value: float = 512.0

    @classmethod
    def from_dict(cls, d: dict) -> "StableAudioProjectionConfig":
        keys = set(cls.__dataclass_fields__)
        return cls(**{k: v for k, v in d.items() if k in keys})


class NumberConditioner(nn.Module):
    """seconds -> one conditioning token: clamp and normalise to [0, 1], [x | sin(2 pi w x) | cos(2 pi w x)]
    with 128 learned frequencies w, then a Linear (``time_positional_embedding.0.weights`` / ``.1``)."""

    def __init__(self, dim, lo, hi, internal_dim=256, dtype=torch.float32, device=None):
        super().__init__()
        self.lo, self.hi = lo, hi
        self.weights = nn.Parameter(torch.randn(internal_dim // 2, dtype=dtype, device=device), requires_grad=False)
        self.linear = nn.Linear(internal_dim + 1, dim, dtype=dtype, device=device)

    def forward(self, seconds: torch.Tensor) -> torch.Tensor:
        x = ((seconds.float().clamp(self.lo, self.hi) - self.lo) / (self.hi - self.lo)).to(self.weights.dtype)[:, None]
        f = x * self.weights[None] * 2 * math.pi
        return self.linear(torch.cat([x, f.sin(), f.cos()], -1))[:, None]               # [B, 1, dim]


class StableAudioProjectionModel(nn.Module):
    def __init__(self, cfg: StableAudioProjectionConfig | None = None, dtype=torch.float32, device=None):
        super().__init__()
        self.config = c = cfg or StableAudioProjectionConfig()
        kw = dict(dtype=dtype, device=device)
        self.text_projection = nn.Linear(c.text_encoder_dim, c.conditioning_dim, **kw) \
            if c.text_encoder_dim != c.conditioning_dim else None
        self.start_number_conditioner = NumberConditioner(c.conditioning_dim, c.min_value, c.max_value, **kw)
        self.end_number_conditioner = NumberConditioner(c.conditioning_dim, c.min_value, c.max_value, **kw)
        for p in self.parameters():
            p.requires_grad_(False)

    def project_text(self, states):
        return states if self.text_projection is None else self.text_projection(states.to(self.text_projection.weight.dtype))

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        loaded = set()
        for n, w in weights:
            tgt = None
            p = n.split(".")
            if p[0] == "text_projection" and self.text_projection is not None:
                tgt = getattr(self.text_projection, p[-1])
            elif p[0] in ("start_number_conditioner", "end_number_conditioner") and p[1] == "time_positional_embedding":
                cond = getattr(self, p[0])
                tgt = cond.weights if p[2] == "0" else getattr(cond.linear, p[-1])
            if tgt is None:
                continue
            tgt.copy_(w.to(tgt.dtype))
            loaded.add(n)
        return loaded
