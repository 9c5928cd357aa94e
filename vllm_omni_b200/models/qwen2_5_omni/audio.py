"""Audio tower of Qwen2.5-Omni (a Whisper-style encoder; the reference takes it from transformers /
vLLM: vllm_omni/model_executor/models/qwen2_5_omni/qwen2_5_omni_thinker.py).

The mel spectrogram [n_mels, T] is cut into chunks of ``2 * n_window`` frames.  Per chunk: Conv1d
(k=3) + GELU, Conv1d (k=3, stride 2) + GELU, sinusoidal positions that restart with the chunk.  The
valid frames of all chunks are encoded by pre-LN transformer layers whose attention stays inside
the chunk (chunks are the batch dimension, the short last chunk carries a key length), then
averaged in pairs over time, layer-normed and projected to the thinker width.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ...diffusion.layers.linear import FusedLinear
from ...ops import fused
from ..qwen3_omni.encoders import EncoderBlock, _block_names


@dataclass
class Qwen25AudioConfig:
    num_mel_bins: int = 128
    d_model: int = 1280
    encoder_layers: int = 32
    encoder_attention_heads: int = 20
    encoder_ffn_dim: int = 5120
    output_dim: int = 3584
    n_window: int = 100
    max_source_positions: int = 1500
    activation_function: str = "gelu"

    @classmethod
    def from_dict(cls, d):
        keys = set(cls.__dataclass_fields__)
        return cls(**{k: v for k, v in d.items() if k in keys})


_BLOCK = _block_names("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.out_proj",
                      "self_attn_layer_norm", "final_layer_norm", "fc1", "fc2")


class Qwen25AudioEncoder(nn.Module):
    def __init__(self, cfg: Qwen25AudioConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        kw = dict(dtype=dtype, device=device)
        D = cfg.d_model
        self.conv1 = nn.Conv1d(cfg.num_mel_bins, D, 3, padding=1, **kw)
        self.conv2 = nn.Conv1d(D, D, 3, stride=2, padding=1, **kw)
        self.layers = nn.ModuleList([EncoderBlock(D, cfg.encoder_attention_heads, cfg.encoder_ffn_dim, 1e-5,
                                                  cfg.activation_function, dtype, device) for _ in range(cfg.encoder_layers)])
        self.ln_post_w = nn.Parameter(torch.ones(D, **kw), requires_grad=False)
        self.ln_post_b = nn.Parameter(torch.zeros(D, **kw), requires_grad=False)
        self.proj = FusedLinear(D, cfg.output_dim, **kw)
        self.audio_bos_eos_token = nn.Parameter(torch.zeros(2, cfg.output_dim, **kw), requires_grad=False)

    def output_length(self, n_frames: int) -> int:
        W = 2 * self.cfg.n_window
        full, tail = divmod(n_frames, W)
        after = full * ((W - 1) // 2 + 1) + (((tail - 1) // 2 + 1) if tail else 0)
        return after // 2                                    # the pair-wise average drops an odd last frame

    @torch.no_grad()
    def forward(self, mel: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        W = 2 * cfg.n_window
        n_mels, T = mel.shape
        n_chunks = max(1, -(-T // W))
        tail = T - (n_chunks - 1) * W
        Lc = W if n_chunks > 1 else tail                          # padded chunk length
        x = mel.to(self.conv1.weight.dtype)
        if n_chunks * Lc != T:
            x = F.pad(x, (0, n_chunks * Lc - T))
        x = x.view(n_mels, n_chunks, Lc).permute(1, 0, 2)           # [chunks, n_mels, Lc]
        valid = torch.ones(n_chunks, 1, Lc, dtype=x.dtype, device=x.device)
        if tail != Lc:
            valid[-1, :, tail:] = 0
        x = F.gelu(self.conv1(x)) * valid                          # padded frames do not leak into the strided conv
        x = F.gelu(self.conv2(x)).transpose(1, 2).contiguous()     # [chunks, t, D]
        t = x.shape[1]
        x = x + self._sinusoid(t, x.shape[-1], x.device).to(x.dtype)[None]
        t_tail = (tail - 1) // 2 + 1
        kv_lens = None
        if t_tail != t:
            kv_lens = torch.full((n_chunks,), t, dtype=torch.int32, device=x.device)
            kv_lens[-1] = t_tail
        for blk in self.layers:
            x = blk(x, kv_lens)
        h = torch.cat([x[:-1].reshape(-1, x.shape[-1]), x[-1, :t_tail]]) if n_chunks > 1 else x[0, :t_tail]
        n = (h.shape[0] // 2) * 2
        h = h[:n].view(n // 2, 2, -1).float().mean(1).to(x.dtype)     # average pairs of frames
        h = fused.norm_modulate(h.contiguous(), weight=self.ln_post_w, bias=self.ln_post_b, eps=1e-5)
        return self.proj(h)

    @staticmethod
    def _sinusoid(n, dim, device):
        half = dim // 2
        inv = torch.exp(-math.log(10000.0) / max(half - 1, 1) * torch.arange(half, device=device).float())
        ang = torch.arange(n, device=device).float()[:, None] * inv[None]
        return torch.cat([ang.sin(), ang.cos()], dim=-1)

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        """Names relative to ``thinker.audio_tower.``."""
        simple = {"conv1.weight": self.conv1.weight, "conv1.bias": self.conv1.bias, "conv2.weight": self.conv2.weight,
                  "conv2.bias": self.conv2.bias, "ln_post.weight": self.ln_post_w, "ln_post.bias": self.ln_post_b,
                  "proj.weight": self.proj.weight, "proj.bias": self.proj.bias,
                  "audio_bos_eos_token.weight": self.audio_bos_eos_token}
        loaded = set()
        for n, w in weights:
            if n in simple:
                simple[n].copy_(w.to(simple[n].dtype))
                loaded.add(n)
            elif n.startswith("layers."):
                p = n.split(".")
                if self.layers[int(p[1])].load(".".join(p[2:]), w, _BLOCK):
                    loaded.add(n)
        return loaded
