"""Encoder of the Qwen3-TTS 12 Hz speech tokenizer: 24 kHz waveform -> [T, 16] codec frames, needed
once per cloned voice for in-context cloning (the reference wraps transformers' ``MimiModel`` and
keeps its first ``encoder_valid_num_quantizers`` codebooks:
vllm_omni/model_executor/models/qwen3_tts/tokenizer_12hz/modeling_qwen3_tts_tokenizer_v2.py:881-973).

Mimi's analysis path: a causal SEANet stack (conv 7, then per ratio 4 / 5 / 6 / 8 a residual unit
[ELU, conv 3, ELU, conv 1] and an ELU + strided conv of kernel 2 x ratio that doubles the width, a
last ELU + conv 3 to the model width), a causal sliding-window transformer (LayerNorm, rotary
attention, GELU MLP, both branches scaled per channel), a stride-2 conv with replicate padding down
to 12.5 frames a second, and a split residual vector quantizer: codebook 0 quantizes its own 1x1
projection of the frame, codebooks 1.. quantize the residuals of ANOTHER projection of the same
frame, each by nearest centroid (``embed_sum / cluster_usage``).

All convolutions pad on the left by (kernel - stride) and on the right just enough to cover the last
frame.  Checkpoint names (under ``encoder.`` in the tokenizer file) are transformers' Mimi names.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn


@dataclass
class MimiEncoderConfig:
    audio_channels: int = 1
    num_filters: int = 64
    kernel_size: int = 7
    last_kernel_size: int = 3
    residual_kernel_size: int = 3
    dilation_growth_rate: int = 2
    num_residual_layers: int = 1
    compress: int = 2
    upsampling_ratios: tuple = (8, 6, 5, 4)
    hidden_size: int = 512
    num_hidden_layers: int = 8
    num_attention_heads: int = 8
    num_key_value_heads: int = 8
    head_dim: int = 64
    intermediate_size: int = 2048
    sliding_window: int = 250
    norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    layer_scale_initial_scale: float = 0.01
    frame_rate: float = 12.5
    sampling_rate: int = 24000
    codebook_size: int = 2048
    codebook_dim: int = 256
    vector_quantization_hidden_dimension: int = 256
    num_quantizers: int = 32
    num_semantic_quantizers: int = 1
    pad_mode: str = "constant"

    @classmethod
    def from_dict(cls, d: dict) -> "MimiEncoderConfig":
        d = dict(d)
        rp = d.get("rope_parameters") or {}
        if "rope_theta" in rp:
            d.setdefault("rope_theta", rp["rope_theta"])
        if d.get("_frame_rate") is not None:              # newer transformers serialise the frame rate under this key
            d.setdefault("frame_rate", d["_frame_rate"])
        keys = set(cls.__dataclass_fields__)
        return cls(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in d.items() if k in keys and v is not None})

    @property
    def encodec_frame_rate(self) -> float:
        return self.sampling_rate / math.prod(self.upsampling_ratios)


class CausalConv(nn.Module):
    """``conv`` with left padding (kernel - stride) and the right padding that completes the last frame."""

    def __init__(self, cin, cout, k, stride=1, dilation=1, bias=True, pad_mode="constant"):
        super().__init__()
        self.conv = nn.Conv1d(cin, cout, k, stride, dilation=dilation, bias=bias)
        self.k_eff, self.stride, self.pad_mode = (k - 1) * dilation + 1, stride, pad_mode
        self.pad = self.k_eff - stride

    def forward(self, x):
        L = x.shape[-1]
        frames = math.ceil((L - self.k_eff + self.pad) / self.stride + 1) - 1
        extra = frames * self.stride + self.k_eff - self.pad - L
        mode = "constant" if self.pad_mode in ("constant", "zero") else self.pad_mode
        return self.conv(F.pad(x, (self.pad, extra), mode=mode))


class ResnetBlock(nn.Module):
    def __init__(self, c: MimiEncoderConfig, dim, dilation):
        super().__init__()
        hid = dim // c.compress
        self.block = nn.ModuleList([nn.ELU(), CausalConv(dim, hid, c.residual_kernel_size, dilation=dilation, pad_mode=c.pad_mode),
                                    nn.ELU(), CausalConv(hid, dim, 1, pad_mode=c.pad_mode)])

    def forward(self, x):
        y = x
        for m in self.block:
            y = m(y)
        return x + y


class MimiLayer(nn.Module):
    def __init__(self, c: MimiEncoderConfig):
        super().__init__()
        D, H, Hkv, Dh = c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim
        self.H, self.Hkv, self.Dh = H, Hkv, Dh
        self.input_layernorm = nn.LayerNorm(D, eps=c.norm_eps)
        self.post_attention_layernorm = nn.LayerNorm(D, eps=c.norm_eps)
        self.q_proj, self.k_proj, self.v_proj = (nn.Linear(D, n * Dh, bias=False) for n in (H, Hkv, Hkv))
        self.o_proj = nn.Linear(H * Dh, D, bias=False)
        self.fc1, self.fc2 = nn.Linear(D, c.intermediate_size, bias=False), nn.Linear(c.intermediate_size, D, bias=False)
        self.attn_scale = nn.Parameter(torch.full((D,), c.layer_scale_initial_scale))
        self.mlp_scale = nn.Parameter(torch.full((D,), c.layer_scale_initial_scale))

    def forward(self, x, cos, sin, mask):
        B, T, _ = x.shape
        h = self.input_layernorm(x)
        q = self.q_proj(h).view(B, T, self.H, self.Dh).transpose(1, 2)
        k = self.k_proj(h).view(B, T, self.Hkv, self.Dh).transpose(1, 2)
        v = self.v_proj(h).view(B, T, self.Hkv, self.Dh).transpose(1, 2)
        rot = lambda t: t * cos + torch.cat([-t[..., self.Dh // 2:], t[..., : self.Dh // 2]], -1) * sin
        q, k = rot(q), rot(k)
        if self.Hkv != self.H:
            k, v = k.repeat_interleave(self.H // self.Hkv, 1), v.repeat_interleave(self.H // self.Hkv, 1)
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=mask).transpose(1, 2).reshape(B, T, -1)
        x = x + self.attn_scale * self.o_proj(o)
        return x + self.mlp_scale * self.fc2(F.gelu(self.fc1(self.post_attention_layernorm(x))))


class Qwen3TTSTokenizerEncoder(nn.Module):
    """fp32; runs once per reference clip."""

    def __init__(self, cfg: MimiEncoderConfig | None = None, valid_quantizers: int = 16, device=None):
        super().__init__()
        self.cfg = c = cfg or MimiEncoderConfig()
        self.valid_quantizers = valid_quantizers
        layers = [CausalConv(c.audio_channels, c.num_filters, c.kernel_size, pad_mode=c.pad_mode)]
        scale = 1
        for ratio in reversed(c.upsampling_ratios):
            dim = scale * c.num_filters
            for j in range(c.num_residual_layers):
                layers.append(ResnetBlock(c, dim, c.dilation_growth_rate ** j))
            layers += [nn.ELU(), CausalConv(dim, dim * 2, ratio * 2, stride=ratio, pad_mode=c.pad_mode)]
            scale *= 2
        layers += [nn.ELU(), CausalConv(scale * c.num_filters, c.hidden_size, c.last_kernel_size, pad_mode=c.pad_mode)]
        self.layers = nn.ModuleList(layers)                                # indices equal transformers' ``encoder.layers``
        self.transformer = nn.ModuleList([MimiLayer(c) for _ in range(c.num_hidden_layers)])
        self.downsample = None
        if c.frame_rate != c.encodec_frame_rate:
            self.downsample = CausalConv(c.hidden_size, c.hidden_size, 2 * int(c.encodec_frame_rate / c.frame_rate), stride=2,
                                         bias=False, pad_mode="replicate")
        Dq = c.vector_quantization_hidden_dimension
        nq = (c.num_semantic_quantizers, c.num_quantizers - c.num_semantic_quantizers)
        self.proj_in = nn.ParameterList([nn.Parameter(torch.randn(Dq, c.hidden_size) * 0.05) for _ in nq])
        self.register_buffer("embed_sum", torch.randn(c.num_quantizers, c.codebook_size, c.codebook_dim))
        self.register_buffer("cluster_usage", torch.ones(c.num_quantizers, c.codebook_size))
        self.inv_freq = 1.0 / (c.rope_theta ** (torch.arange(0, c.head_dim, 2, dtype=torch.float32) / c.head_dim))
        self.to(device=device, dtype=torch.float32)
        for p in self.parameters():
            p.requires_grad_(False)

    @property
    def downsample_rate(self) -> int:
        return int(round(self.cfg.sampling_rate / self.cfg.frame_rate))

    @torch.no_grad()
    def features(self, wav: torch.Tensor) -> torch.Tensor:
        """wav [B, T] -> frame embeddings [B, hidden, T']."""
        c = self.cfg
        x = wav.float()[:, None]
        for m in self.layers:
            x = m(x)
        x = x.transpose(1, 2)
        T = x.shape[1]
        i = torch.arange(T, device=x.device)
        ang = i.float()[:, None] * self.inv_freq.to(x.device)[None]
        cos, sin = torch.cat([ang.cos(), ang.cos()], -1)[None, None], torch.cat([ang.sin(), ang.sin()], -1)[None, None]
        mask = (i[None, :] <= i[:, None]) & (i[:, None] - i[None, :] < c.sliding_window)
        for layer in self.transformer:
            x = layer(x, cos, sin, mask)
        x = x.transpose(1, 2)
        return self.downsample(x) if self.downsample is not None else x

    @torch.no_grad()
    def quantize(self, emb: torch.Tensor, num_quantizers: int | None = None) -> torch.Tensor:
        """emb [B, hidden, T'] -> codes [B, K, T']."""
        c = self.cfg
        K = num_quantizers or self.valid_quantizers
        tables = self.embed_sum / self.cluster_usage.clamp(min=1e-5)[..., None]
        codes = []
        for grp, (lo, hi) in enumerate(((0, c.num_semantic_quantizers), (c.num_semantic_quantizers, c.num_quantizers))):
            res = torch.einsum("qd,bdt->btq", self.proj_in[grp], emb)               # [B, T', Dq]
            for g in range(lo, min(hi, K)):
                idx = torch.cdist(res.reshape(1, -1, res.shape[-1]), tables[g][None])[0].argmin(-1).view(res.shape[:2])
                res = res - tables[g][idx]
                codes.append(idx)
        return torch.stack(codes, dim=1)

    @torch.no_grad()
    def encode(self, wav: torch.Tensor) -> torch.Tensor:
        """One clip [T] at the tokenizer's sampling rate -> frames [T', valid_quantizers] (int64)."""
        wav = wav.reshape(1, -1).to(self.embed_sum.device)
        codes = self.quantize(self.features(wav))[0]
        n = -(-wav.shape[1] // self.downsample_rate)
        return codes[:, :n].t().contiguous()

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        """Names relative to the tokenizer's ``encoder.`` module (transformers' ``MimiModel``)."""
        c = self.cfg
        loaded = set()
        for n, w in weights:
            p = n.split(".")
            tgt = None
            if p[0] == "encoder" and p[1] == "layers":
                m = self.layers[int(p[2])]
                if isinstance(m, ResnetBlock) and p[3] == "block":
                    tgt = getattr(m.block[int(p[4])].conv, p[-1])
                elif isinstance(m, CausalConv) and p[3] == "conv":
                    tgt = getattr(m.conv, p[-1])
            elif p[0] == "encoder_transformer" and p[1] == "layers":
                layer, rest = self.transformer[int(p[2])], ".".join(p[3:])
                tgt = {"self_attn.q_proj.weight": layer.q_proj.weight, "self_attn.k_proj.weight": layer.k_proj.weight,
                       "self_attn.v_proj.weight": layer.v_proj.weight, "self_attn.o_proj.weight": layer.o_proj.weight,
                       "mlp.fc1.weight": layer.fc1.weight, "mlp.fc2.weight": layer.fc2.weight,
                       "input_layernorm.weight": layer.input_layernorm.weight, "input_layernorm.bias": layer.input_layernorm.bias,
                       "post_attention_layernorm.weight": layer.post_attention_layernorm.weight,
                       "post_attention_layernorm.bias": layer.post_attention_layernorm.bias,
                       "self_attn_layer_scale.scale": layer.attn_scale, "mlp_layer_scale.scale": layer.mlp_scale}.get(rest)
            elif n == "downsample.conv.weight" and self.downsample is not None:
                tgt = self.downsample.conv.weight
            elif p[0] == "quantizer":
                grp = 0 if p[1].startswith("semantic") else 1
                off = 0 if grp == 0 else c.num_semantic_quantizers
                if p[2] == "input_proj":
                    tgt, w = self.proj_in[grp], w.reshape(w.shape[0], -1)
                elif p[2] == "layers" and p[4] == "codebook" and p[5] in ("embed_sum", "cluster_usage"):
                    tgt = getattr(self, p[5])[off + int(p[3])]
            if tgt is None:
                continue
            tgt.copy_(w.to(tgt.dtype).reshape(tgt.shape))
            loaded.add(n)
        return loaded
