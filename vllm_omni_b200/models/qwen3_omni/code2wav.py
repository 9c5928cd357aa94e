"""Qwen3-Omni code2wav stage: codec frames [T, G] -> 24 kHz waveform.

Sum of per-codebook embeddings -> a few sliding-window transformer layers -> transposed-conv
up-sampling stack with SnakeBeta activations (total factor = prod(upsample_rates) *
prod(upsampling_ratios)).  Long sequences are decoded in chunks of ``chunk_size`` frames with
``left_context`` frames of overlap whose samples are discarded
(vllm_omni/model_executor/models/qwen3_omni/qwen3_omni_code2wav.py, chunked_decode).
A one-shot ("generation") stage: no sampling, no KV cache.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from ...ops.attention import attention_reference
from ..base import StageModel
from .config import Code2WavConfig, Qwen3OmniConfig


class SnakeBeta(nn.Module):
    def __init__(self, ch, dtype, device):
        super().__init__()
        self.alpha = nn.Parameter(torch.zeros(ch, dtype=dtype, device=device), requires_grad=False)
        self.beta = nn.Parameter(torch.zeros(ch, dtype=dtype, device=device), requires_grad=False)

    def forward(self, x):           # x: [B, C, T]
        a = self.alpha.float().exp()[None, :, None]
        b = self.beta.float().exp()[None, :, None]
        xf = x.float()
        return (xf + (1.0 / (b + 1e-9)) * torch.sin(xf * a).pow(2)).to(x.dtype)


class ResUnit(nn.Module):
    def __init__(self, ch, dilation, dtype, device):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.act1, self.act2 = SnakeBeta(ch, dtype, device), SnakeBeta(ch, dtype, device)
        self.conv1 = nn.Conv1d(ch, ch, 7, dilation=dilation, padding=0, **kw)
        self.conv2 = nn.Conv1d(ch, ch, 1, **kw)
        self.pad = 6 * dilation

    def forward(self, x):
        h = self.conv1(F.pad(self.act1(x), (self.pad, 0)))          # causal
        return x + self.conv2(self.act2(h))


class UpBlock(nn.Module):
    def __init__(self, cin, cout, rate, dtype, device):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.act = SnakeBeta(cin, dtype, device)
        self.up = nn.ConvTranspose1d(cin, cout, 2 * rate, stride=rate, **kw)
        self.rate = rate
        self.res = nn.ModuleList([ResUnit(cout, d, dtype, device) for d in (1, 3, 9)])

    def forward(self, x):
        y = self.up(self.act(x))
        y = y[..., :x.shape[-1] * self.rate]                          # causal trim
        for r in self.res:
            y = r(y)
        return y


class WindowBlock(nn.Module):
    def __init__(self, cfg: Code2WavConfig, dtype, device):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        D = cfg.hidden_size
        self.heads, self.window = cfg.num_attention_heads, cfg.sliding_window
        self.n1 = nn.Parameter(torch.ones(D, **kw), requires_grad=False)
        self.n2 = nn.Parameter(torch.ones(D, **kw), requires_grad=False)
        self.qkv = nn.Linear(D, 3 * D, bias=False, **kw)
        self.o = nn.Linear(D, D, bias=False, **kw)
        self.gate_up = nn.Linear(D, 2 * cfg.intermediate_size, bias=False, **kw)
        self.down = nn.Linear(cfg.intermediate_size, D, bias=False, **kw)

    @staticmethod
    def _rms(x, w):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()).to(x.dtype)

    def forward(self, x):           # [B, T, D]
        B, T, D = x.shape
        qkv = self.qkv(self._rms(x, self.n1)).view(B, T, 3, self.heads, D // self.heads)
        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
        i = torch.arange(T, device=x.device)
        mask = (i[None, :] <= i[:, None]) & (i[:, None] - i[None, :] < self.window)
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=mask).transpose(1, 2).reshape(B, T, D)
        x = x + self.o(o)
        h = self.gate_up(self._rms(x, self.n2))
        F_ = h.shape[-1] // 2
        return x + self.down(F.silu(h[..., :F_]) * h[..., F_:])


class Qwen3OmniCode2Wav(StageModel):
    engine_output_type = "audio"
    is_generation_model = True

    def __init__(self, cfg: Qwen3OmniConfig, dtype=torch.bfloat16, device=None):
        super().__init__(None, dtype, device)
        c = self.c = cfg.code2wav
        kw = dict(dtype=dtype, device=device)
        self.code_embedding = nn.Parameter(torch.empty(c.num_quantizers, c.codebook_size, c.hidden_size, **kw)
                                           .normal_(0, 0.02), requires_grad=False)
        self.pre = nn.ModuleList([WindowBlock(c, dtype, device) for _ in range(c.num_hidden_layers)])
        self.pre_up = nn.ModuleList()
        ch = c.hidden_size
        for r in c.upsampling_ratios:
            self.pre_up.append(nn.ConvTranspose1d(ch, ch, r, stride=r, **kw))
        self.conv_in = nn.Conv1d(ch, c.decoder_dim, 7, padding=0, **kw)
        ups, cin = [], c.decoder_dim
        for r in c.upsample_rates:
            ups.append(UpBlock(cin, max(cin // 2, 8), r, dtype, device))
            cin = max(cin // 2, 8)
        self.ups = nn.ModuleList(ups)
        self.act_out = SnakeBeta(cin, dtype, device)
        self.conv_out = nn.Conv1d(cin, 1, 7, padding=0, **kw)

    @torch.no_grad()
    def decode(self, codes: torch.Tensor) -> torch.Tensor:
        """codes: [B, G, T] int64 -> waveform [B, T * total_upsample] in [-1, 1]."""
        c = self.c
        B, G, T = codes.shape
        x = sum(self.code_embedding[g][codes[:, g].clamp(0, c.codebook_size - 1)] for g in range(G))   # [B, T, D]
        for blk in self.pre:
            x = blk(x)
        x = x.transpose(1, 2)
        for up in self.pre_up:
            x = up(x)
        x = self.conv_in(F.pad(x, (6, 0)))
        for up in self.ups:
            x = up(x)
        x = self.conv_out(F.pad(self.act_out(x), (6, 0)))
        return torch.tanh(x.float())[:, 0]

    @torch.no_grad()
    def chunked_decode(self, codes: torch.Tensor, chunk_size=None, left_context=None) -> torch.Tensor:
        c = self.c
        chunk_size = chunk_size or c.chunk_size
        left = c.left_context if left_context is None else left_context
        T = codes.shape[-1]
        up = c.total_upsample
        if T == 0:
            return torch.zeros(codes.shape[0], 0, device=codes.device)
        outs, start = [], 0
        while start < T:
            end = min(T, start + chunk_size)
            ctx = min(left, start)
            wav = self.decode(codes[..., start - ctx:end])
            outs.append(wav[..., ctx * up:])
            start = end
        return torch.cat(outs, dim=-1)

    def generate_for(self, req, start, n):
        info = req.additional_information
        codes = info.get("codes")
        if codes is None:                       # token ids carry a flattened [T * G] code list
            G = self.c.num_quantizers
            ids = torch.tensor(req.prompt_token_ids[start:start + n], dtype=torch.long)
            codes = ids[: (ids.numel() // G) * G].view(-1, G)
        codes = torch.as_tensor(codes).long().to(self.code_embedding.device)
        if codes.dim() == 2:                    # [T, G] -> [1, G, T]
            codes = codes.t()[None]
        ctx = int(info.get("left_context_frames", 0))
        wav = self.chunked_decode(codes)
        if ctx:
            wav = wav[..., ctx * self.c.total_upsample:]
        return {"audio": wav[0].float(), "sample_rate": self.c.sample_rate}
