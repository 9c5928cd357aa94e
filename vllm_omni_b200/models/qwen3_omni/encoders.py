"""Audio and vision towers of the thinker (vllm_omni/model_executor/models/qwen3_omni/
qwen3_omni_moe_thinker.py: audio tower, ViT with deep-stack merger).  Both are encoder-only
transformers; their linear layers and attention go through the same sm_100a ops as the
decoders (``FusedLinear`` / ``attention``), the convolution stems use PyTorch convs."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from ...diffusion.layers.linear import FusedLinear
from ...ops import fused
from ...ops.attention import attention, attention_reference
from .config import AudioEncoderConfig, VisionEncoderConfig


def _mha(q, k, v):
    """[B, S, H, D] non-causal attention; the tcgen05 kernel needs D == 128, other head sizes
    take the reference formula (small towers only)."""
    if q.is_cuda and q.shape[-1] == 128 and q.dtype == torch.bfloat16:
        return attention(q, k, v)
    return attention_reference(q, k, v)


class EncoderBlock(nn.Module):
    def __init__(self, dim, heads, ffn, dtype, device):
        super().__init__()
        self.heads = heads
        self.ln1_w = nn.Parameter(torch.ones(dim, dtype=dtype, device=device), requires_grad=False)
        self.ln1_b = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device), requires_grad=False)
        self.ln2_w = nn.Parameter(torch.ones(dim, dtype=dtype, device=device), requires_grad=False)
        self.ln2_b = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device), requires_grad=False)
        self.qkv = FusedLinear(dim, 3 * dim, dtype=dtype, device=device)
        self.proj = FusedLinear(dim, dim, dtype=dtype, device=device)
        self.fc1 = FusedLinear(dim, ffn, dtype=dtype, device=device)
        self.fc2 = FusedLinear(ffn, dim, dtype=dtype, device=device)

    def forward(self, x):           # x: [B, S, D]
        B, S, D = x.shape
        h = fused.norm_modulate(x, weight=self.ln1_w, bias=self.ln1_b, eps=1e-5)
        qkv = self.qkv(h).view(B, S, 3, self.heads, D // self.heads)
        o = _mha(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]).reshape(B, S, D)
        x = self.proj(o.contiguous(), residual=x)
        h = fused.norm_modulate(x, weight=self.ln2_w, bias=self.ln2_b, eps=1e-5)
        return self.fc2(self.fc1(h, act="gelu_tanh"), residual=x)


class AudioEncoder(nn.Module):
    """mel [n_mels, T] -> [T/8..., output_dim]: three stride-2 2-D convs over (mel, time), then
    windowed encoder blocks, then a two-layer projection."""

    def __init__(self, cfg: AudioEncoderConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        c = cfg.downsample_hidden_size
        kw = dict(dtype=dtype, device=device)
        self.conv1 = nn.Conv2d(1, c, 3, 2, 1, **kw)
        self.conv2 = nn.Conv2d(c, c, 3, 2, 1, **kw)
        self.conv3 = nn.Conv2d(c, c, 3, 2, 1, **kw)
        f = cfg.num_mel_bins
        for _ in range(3):
            f = (f + 1) // 2
        self.conv_out = FusedLinear(c * f, cfg.d_model, bias=False, dtype=dtype, device=device)
        self.blocks = nn.ModuleList([EncoderBlock(cfg.d_model, cfg.encoder_attention_heads, cfg.encoder_ffn_dim,
                                                  dtype, device) for _ in range(cfg.encoder_layers)])
        self.ln_w = nn.Parameter(torch.ones(cfg.d_model, **kw), requires_grad=False)
        self.ln_b = nn.Parameter(torch.zeros(cfg.d_model, **kw), requires_grad=False)
        self.proj1 = FusedLinear(cfg.d_model, cfg.d_model, dtype=dtype, device=device)
        self.proj2 = FusedLinear(cfg.d_model, cfg.output_dim, dtype=dtype, device=device)

    def output_length(self, n_frames: int) -> int:
        for _ in range(3):
            n_frames = (n_frames + 1) // 2
        return n_frames

    def forward(self, mel: torch.Tensor) -> torch.Tensor:
        x = mel.to(self.conv1.weight.dtype)[None, None]                  # [1, 1, n_mels, T]
        x = F.gelu(self.conv1(x))
        x = F.gelu(self.conv2(x))
        x = F.gelu(self.conv3(x))                                        # [1, C, F', T']
        _, C, Fq, Tq = x.shape
        x = x.permute(0, 3, 1, 2).reshape(1, Tq, C * Fq).contiguous()
        x = self.conv_out(x)
        pos = self._sinusoid(Tq, x.shape[-1], x.device).to(x.dtype)
        x = x + pos[None]
        # windowed attention: windows are independent sequences -> fold them into the batch
        W = self.cfg.n_window * 2
        pad = (-Tq) % W
        if pad:
            x = F.pad(x, (0, 0, 0, pad))
        xb = x.view(-1, W, x.shape[-1]).contiguous()
        for blk in self.blocks:
            xb = blk(xb)
        x = xb.view(1, -1, xb.shape[-1])[:, :Tq]
        x = fused.norm_modulate(x.contiguous(), weight=self.ln_w, bias=self.ln_b, eps=1e-5)
        return self.proj2(self.proj1(x, act="gelu_tanh"))[0]

    @staticmethod
    def _sinusoid(n, dim, device):
        half = dim // 2
        inv = torch.exp(-math.log(10000.0) * torch.arange(half, device=device).float() / max(half - 1, 1))
        ang = torch.arange(n, device=device).float()[:, None] * inv[None]
        return torch.cat([ang.sin(), ang.cos()], dim=-1)


class VisionEncoder(nn.Module):
    """pixels [T, C, H, W] -> merged patch embeddings [T' * (H/p/m) * (W/p/m), out_hidden]."""

    def __init__(self, cfg: VisionEncoderConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        kw = dict(dtype=dtype, device=device)
        pd = cfg.in_channels * cfg.temporal_patch_size * cfg.patch_size * cfg.patch_size
        self.patch_embed = FusedLinear(pd, cfg.hidden_size, dtype=dtype, device=device)
        self.blocks = nn.ModuleList([EncoderBlock(cfg.hidden_size, cfg.num_heads, cfg.intermediate_size, dtype, device)
                                     for _ in range(cfg.depth)])
        m = cfg.spatial_merge_size ** 2
        self.ln_w = nn.Parameter(torch.ones(cfg.hidden_size, **kw), requires_grad=False)
        self.ln_b = nn.Parameter(torch.zeros(cfg.hidden_size, **kw), requires_grad=False)
        self.merge1 = FusedLinear(cfg.hidden_size * m, cfg.hidden_size * m, dtype=dtype, device=device)
        self.merge2 = FusedLinear(cfg.hidden_size * m, cfg.out_hidden_size, dtype=dtype, device=device)

    def grid(self, T, H, W):
        c = self.cfg
        return max(1, T // c.temporal_patch_size), H // c.patch_size, W // c.patch_size

    def forward(self, pixels: torch.Tensor) -> tuple[torch.Tensor, tuple]:
        c = self.cfg
        T, C, H, W = pixels.shape
        if T % c.temporal_patch_size:
            pixels = torch.cat([pixels, pixels[-1:].expand(c.temporal_patch_size - T % c.temporal_patch_size, -1, -1, -1)])
            T = pixels.shape[0]
        gt, gh, gw = self.grid(T, H, W)
        p, m = c.patch_size, c.spatial_merge_size
        x = pixels[:, :, :gh * p, :gw * p].reshape(gt, c.temporal_patch_size, C, gh // m, m, p, gw // m, m, p)
        # order patches so that the m x m merge group is contiguous
        x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8).reshape(gt * gh * gw, -1)
        x = self.patch_embed(x.to(self.ln_w.dtype).contiguous())[None]
        for blk in self.blocks:
            x = blk(x)
        x = fused.norm_modulate(x.contiguous(), weight=self.ln_w, bias=self.ln_b, eps=1e-6)
        x = x.reshape(-1, c.hidden_size * m * m)
        return self.merge2(self.merge1(x, act="gelu_tanh")), (gt, gh // m, gw // m)
