"""T5 / UMT5 encoder as a prompt encoder (FLUX and SD3 use T5-v1.1-XXL, Stable Audio T5-base, Wan UMT5-XXL; the
reference instantiates ``transformers.T5EncoderModel`` inside its pipelines, e.g.
vllm_omni/diffusion/models/flux/pipeline_flux.py, stable_audio/pipeline_stable_audio.py).

Pre-norm blocks with scale-only RMS norms; attention WITHOUT the 1/sqrt(d) factor and with a learned
additive bias per (head, bucketed relative position) that block 0 owns and every block reuses (UMT5: every
block has its own table); a
feed-forward that is either ReLU (``wi``/``wo``) or gated GELU (``wi_0``/``wi_1``/``wo``).  The bias
table is looked up once per sequence length and cached.  The attention core is torch's fused SDPA with
that bias as the additive mask: the encoder runs once per request, outside the denoising loop.

Checkpoint names: ``shared.weight`` (or ``encoder.embed_tokens.weight``), ``encoder.block.N.layer.0.
SelfAttention.{q,k,v,o}.weight``, ``...relative_attention_bias.weight`` (block 0), ``encoder.block.N.
layer.0|1.layer_norm.weight``, ``encoder.block.N.layer.1.DenseReluDense.*``, ``encoder.final_layer_norm.weight``.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ....ops import fused
from ...layers.linear import FusedLinear


@dataclass
class T5Config:
    vocab_size: int = 32128
    d_model: int = 4096
    d_kv: int = 64
    d_ff: int = 10240
    num_layers: int = 24
    num_heads: int = 64
    relative_attention_num_buckets: int = 32
    relative_attention_max_distance: int = 128
    layer_norm_epsilon: float = 1e-6
    feed_forward_proj: str = "gated-gelu"          # "relu" | "gated-gelu"
    per_layer_bias: bool = False                   # UMT5 (Wan's encoder): every block owns a relative-position bias table

    @classmethod
    def from_dict(cls, d: dict) -> "T5Config":
        d = dict(d)
        if d.get("model_type") == "umt5" or any("UMT5" in a for a in d.get("architectures") or []):
            d.setdefault("per_layer_bias", True)
        keys = set(cls.__dataclass_fields__)
        return cls(**{k: v for k, v in d.items() if k in keys})

    @property
    def gated(self) -> bool:
        return self.feed_forward_proj.startswith("gated")


def relative_position_bucket(rel: torch.Tensor, num_buckets: int, max_distance: int) -> torch.Tensor:
    """Bidirectional bucketing of key_position - query_position: half of the buckets per sign; within a
    sign the first half is exact, the rest logarithmic up to ``max_distance``."""
    nb = num_buckets // 2
    out = (rel > 0).long() * nb
    rel = rel.abs()
    max_exact = nb // 2
    large = max_exact + (torch.log(rel.float().clamp(min=1) / max_exact) / math.log(max_distance / max_exact)
                         * (nb - max_exact)).long()
    large = torch.minimum(large, torch.full_like(large, nb - 1))
    return out + torch.where(rel < max_exact, rel, large)


class T5Block(nn.Module):
    def __init__(self, c: T5Config, dtype, device):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        inner = c.num_heads * c.d_kv
        self.c = c
        self.norm1 = nn.Parameter(torch.ones(c.d_model, **kw), requires_grad=False)
        self.norm2 = nn.Parameter(torch.ones(c.d_model, **kw), requires_grad=False)
        self.qkv = FusedLinear(c.d_model, 3 * inner, bias=False, **kw)
        self.o = FusedLinear(inner, c.d_model, bias=False, **kw)
        self.wi = FusedLinear(c.d_model, (2 if c.gated else 1) * c.d_ff, bias=False, **kw)
        self.wo = FusedLinear(c.d_ff, c.d_model, bias=False, **kw)

    def forward(self, x, bias):                     # x [B, L, D]; bias [B or 1, H, L, L] additive (fp32)
        c = self.c
        B, L, _ = x.shape
        h = fused.norm_modulate(x, weight=self.norm1, rms=True, eps=c.layer_norm_epsilon)
        q, k, v = self.qkv(h).view(B, L, 3, c.num_heads, c.d_kv).permute(2, 0, 3, 1, 4)
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=bias.to(q.dtype), scale=1.0)
        x = self.o(o.transpose(1, 2).reshape(B, L, -1).contiguous(), residual=x)
        h = fused.norm_modulate(x, weight=self.norm2, rms=True, eps=c.layer_norm_epsilon)
        u = self.wi(h)
        if c.gated:
            g, up = u.chunk(2, dim=-1)
            u = F.gelu(g.float(), approximate="tanh").to(u.dtype) * up
        else:
            u = F.relu(u)
        return self.wo(u.contiguous(), residual=x)


class T5Encoder(nn.Module):
    def __init__(self, cfg: T5Config, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = c = cfg
        kw = dict(dtype=dtype, device=device)
        self.embed = nn.Parameter(torch.empty(c.vocab_size, c.d_model, **kw).normal_(0, 1.0), requires_grad=False)
        self.rel_bias = nn.Parameter(torch.zeros(c.num_layers if c.per_layer_bias else 1, c.relative_attention_num_buckets,
                                                 c.num_heads, **kw), requires_grad=False)
        self.blocks = nn.ModuleList([T5Block(c, dtype, device) for _ in range(c.num_layers)])
        self.final_norm = nn.Parameter(torch.ones(c.d_model, **kw), requires_grad=False)
        self._bias_cache: dict[int, torch.Tensor] = {}

    def position_bias(self, L: int) -> torch.Tensor:
        b = self._bias_cache.get(L)
        if b is None or b.device != self.rel_bias.device:
            pos = torch.arange(L, device=self.rel_bias.device)
            bucket = relative_position_bucket(pos[None, :] - pos[:, None], self.cfg.relative_attention_num_buckets,
                                              self.cfg.relative_attention_max_distance)
            b = self.rel_bias.float()[:, bucket].permute(0, 3, 1, 2)[:, None].contiguous()   # [tables, 1, H, L, L]
            self._bias_cache = {L: b}
        return b

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, attention_mask: torch.Tensor | None = None) -> torch.Tensor:
        """input_ids [B, L] -> last hidden state [B, L, d_model]; padded keys are masked out."""
        B, L = input_ids.shape
        x = self.embed[input_ids]
        bias = self.position_bias(L)
        if attention_mask is not None:
            neg = torch.finfo(torch.float32).min
            bias = bias + ((1.0 - attention_mask[:, None, None, :].float()) * neg)[None]
        for i, blk in enumerate(self.blocks):
            x = blk(x, bias[i if self.cfg.per_layer_bias else 0])
        return fused.norm_modulate(x.contiguous(), weight=self.final_norm, rms=True, eps=self.cfg.layer_norm_epsilon)

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        c = self.cfg
        inner = c.num_heads * c.d_kv
        loaded = set()
        for n, w in weights:
            p = n.split(".")
            tgt, sl = None, None
            if n in ("shared.weight", "encoder.embed_tokens.weight"):
                tgt = self.embed
            elif n == "encoder.final_layer_norm.weight":
                tgt = self.final_norm
            elif n.startswith("encoder.block."):
                blk = self.blocks[int(p[2])]
                rest = ".".join(p[3:])
                if rest.startswith("layer.0.SelfAttention.") and p[6] in ("q", "k", "v"):
                    i = "qkv".index(p[6])
                    tgt, sl = blk.qkv.weight, (i * inner, (i + 1) * inner)
                elif rest == "layer.0.SelfAttention.o.weight":
                    tgt = blk.o.weight
                elif rest == "layer.0.SelfAttention.relative_attention_bias.weight":
                    tgt = self.rel_bias[int(p[2]) if c.per_layer_bias else 0]
                    self._bias_cache = {}
                elif rest == "layer.0.layer_norm.weight":
                    tgt = blk.norm1
                elif rest == "layer.1.layer_norm.weight":
                    tgt = blk.norm2
                elif rest == "layer.1.DenseReluDense.wi_0.weight":
                    tgt, sl = blk.wi.weight, (0, c.d_ff)
                elif rest == "layer.1.DenseReluDense.wi_1.weight":
                    tgt, sl = blk.wi.weight, (c.d_ff, 2 * c.d_ff)
                elif rest == "layer.1.DenseReluDense.wi.weight":
                    tgt = blk.wi.weight
                elif rest == "layer.1.DenseReluDense.wo.weight":
                    tgt = blk.wo.weight
            if tgt is None:
                continue
            dst = tgt if sl is None else tgt[sl[0]:sl[1]]
            dst.copy_(w.to(dst.dtype))
            loaded.add(n)
        return loaded


class T5PromptEncoder:
    """texts -> (states [B, max_len, d_model], mask [B, max_len]), padded to ``max_len`` like the
    diffusers pipelines do.  FLUX and SD3 run the encoder without a mask and hand every position to the
    DiT (the returned mask is all ones); ``zero_padding`` (Stable Audio) masks padded keys inside the
    encoder, zeroes their states and returns the tokenizer's mask."""

    def __init__(self, model: T5Encoder, tokenizer, max_len: int = 512, zero_padding: bool = False):
        self.model, self.tokenizer, self.max_len, self.zero_padding = model, tokenizer, max_len, zero_padding

    @classmethod
    def from_pretrained(cls, model_path: str, subfolder: str, tokenizer_subfolder: str, dtype, device, max_len=512, **kw):
        from transformers import AutoTokenizer
        with open(os.path.join(model_path, subfolder, "config.json")) as f:
            cfg = T5Config.from_dict(json.load(f))
        tok = AutoTokenizer.from_pretrained(os.path.join(model_path, tokenizer_subfolder))
        return cls(T5Encoder(cfg, dtype, device), tok, max_len, **kw)

    def load_weights(self, weights) -> set:
        return self.model.load_weights(weights)

    @torch.no_grad()
    def __call__(self, texts, device, dtype=None, max_len: int | None = None):
        L = min(int(max_len or self.max_len), self.max_len)
        enc = self.tokenizer(list(texts), padding="max_length", max_length=L, truncation=True, return_tensors="pt")
        ids, mask = enc["input_ids"].to(device), enc["attention_mask"].to(device)
        out = self.model(ids, mask if self.zero_padding else None)
        if self.zero_padding:
            out = out * mask[..., None].to(out.dtype)
        else:
            mask = torch.ones_like(mask)             # FLUX / SD3: the padded positions are real keys of the DiT
        return (out if dtype is None else out.to(dtype)), mask
