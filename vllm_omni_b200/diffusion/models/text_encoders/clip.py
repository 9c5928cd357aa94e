"""CLIP text encoder as a prompt encoder: FLUX takes its pooled vector, SD3 the pooled vectors of
two CLIP towers (with projection) plus their penultimate hidden states (the reference instantiates
``transformers.CLIPTextModel`` / ``CLIPTextModelWithProjection`` inside its pipelines, e.g.
vllm_omni/diffusion/models/flux/pipeline_flux.py, sd3/pipeline_sd3.py).

Token + learned position embeddings, pre-LayerNorm blocks with CAUSAL attention and biased
projections, quick-GELU (x * sigmoid(1.702 x)) or GELU feed-forward, a final LayerNorm; the pooled
vector is the final state at the end-of-text token (the first occurrence of ``eos_token_id``, or, for
the original checkpoints whose config says ``eos_token_id == 2``, the position of the largest token
id), optionally through a bias-free ``text_projection``.

Checkpoint names: ``text_model.embeddings.{token_embedding,position_embedding}.weight``,
``text_model.encoder.layers.N.{layer_norm1,layer_norm2,self_attn.{q,k,v,out}_proj,mlp.fc1,mlp.fc2}.*``,
``text_model.final_layer_norm.*``, ``text_projection.weight``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ...layers.linear import FusedLinear


@dataclass
class CLIPTextConfig:
    vocab_size: int = 49408
    hidden_size: int = 768
    intermediate_size: int = 3072
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    max_position_embeddings: int = 77
    hidden_act: str = "quick_gelu"
    layer_norm_eps: float = 1e-5
    eos_token_id: int = 2
    projection_dim: int | None = None               # set: pooled vector goes through ``text_projection``

    @classmethod
    def from_dict(cls, d: dict) -> "CLIPTextConfig":
        keys = set(cls.__dataclass_fields__)
        c = cls(**{k: v for k, v in d.items() if k in keys})
        if "CLIPTextModelWithProjection" not in (d.get("architectures") or []) and not d.get("_with_projection"):
            c.projection_dim = None
        return c


class CLIPLayer(nn.Module):
    def __init__(self, c: CLIPTextConfig, dtype, device):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        D = c.hidden_size
        self.heads, self.act = c.num_attention_heads, c.hidden_act
        self.ln1 = nn.LayerNorm(D, eps=c.layer_norm_eps, **kw)
        self.ln2 = nn.LayerNorm(D, eps=c.layer_norm_eps, **kw)
        self.qkv = FusedLinear(D, 3 * D, **kw)
        self.out = FusedLinear(D, D, **kw)
        self.fc1 = FusedLinear(D, c.intermediate_size, **kw)
        self.fc2 = FusedLinear(c.intermediate_size, D, **kw)

    def forward(self, x):
        B, L, D = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(B, L, 3, self.heads, D // self.heads).permute(2, 0, 3, 1, 4)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = self.out(o.transpose(1, 2).reshape(B, L, D).contiguous(), residual=x)
        h = self.fc1(self.ln2(x))
        if self.act == "quick_gelu":
            h = h * torch.sigmoid(1.702 * h.float()).to(h.dtype)
        else:
            h = F.gelu(h.float()).to(h.dtype)
        return self.fc2(h, residual=x)


class CLIPTextEncoder(nn.Module):
    def __init__(self, cfg: CLIPTextConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = c = cfg
        kw = dict(dtype=dtype, device=device)
        self.token_embedding = nn.Parameter(torch.empty(c.vocab_size, c.hidden_size, **kw).normal_(0, 0.02), requires_grad=False)
        self.position_embedding = nn.Parameter(torch.empty(c.max_position_embeddings, c.hidden_size, **kw).normal_(0, 0.01),
                                               requires_grad=False)
        self.layers = nn.ModuleList([CLIPLayer(c, dtype, device) for _ in range(c.num_hidden_layers)])
        self.final_layer_norm = nn.LayerNorm(c.hidden_size, eps=c.layer_norm_eps, **kw)
        self.text_projection = FusedLinear(c.hidden_size, c.projection_dim, bias=False, **kw) if c.projection_dim else None
        for p in self.parameters():
            p.requires_grad_(False)

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor):
        """Returns (final states [B, L, D] after the last LayerNorm, pooled [B, D or projection_dim],
        penultimate block output [B, L, D] before the final LayerNorm)."""
        c = self.cfg
        B, L = input_ids.shape
        x = self.token_embedding[input_ids] + self.position_embedding[:L][None]
        penultimate = x
        for i, layer in enumerate(self.layers):
            if i == len(self.layers) - 1:
                penultimate = x
            x = layer(x)
        last = self.final_layer_norm(x)
        if c.eos_token_id == 2:
            eos = input_ids.argmax(-1)
        else:
            eos = (input_ids == c.eos_token_id).int().argmax(-1)
        pooled = last[torch.arange(B, device=last.device), eos]
        if self.text_projection is not None:
            pooled = self.text_projection(pooled.contiguous())
        return last, pooled, penultimate

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        D = self.cfg.hidden_size
        loaded = set()
        for n, w in weights:
            p = n.split(".")
            tgt, sl = None, None
            if n == "text_model.embeddings.token_embedding.weight":
                tgt = self.token_embedding
            elif n == "text_model.embeddings.position_embedding.weight":
                tgt = self.position_embedding
            elif n.startswith("text_model.final_layer_norm."):
                tgt = getattr(self.final_layer_norm, p[-1])
            elif n == "text_projection.weight" and self.text_projection is not None:
                tgt = self.text_projection.weight
            elif n.startswith("text_model.encoder.layers."):
                layer, leaf = self.layers[int(p[3])], p[-1]
                if p[4] == "self_attn" and p[5] in ("q_proj", "k_proj", "v_proj"):
                    i = ("q_proj", "k_proj", "v_proj").index(p[5])
                    tgt, sl = getattr(layer.qkv, leaf), (i * D, (i + 1) * D)
                elif p[4] == "self_attn" and p[5] == "out_proj":
                    tgt = getattr(layer.out, leaf)
                elif p[4] in ("layer_norm1", "layer_norm2"):
                    tgt = getattr(layer.ln1 if p[4] == "layer_norm1" else layer.ln2, leaf)
                elif p[4] == "mlp":
                    tgt = getattr(getattr(layer, p[5]), leaf)
            if tgt is None:
                continue
            dst = tgt if sl is None else tgt[sl[0]:sl[1]]
            dst.copy_(w.to(dst.dtype))
            loaded.add(n)
        return loaded


class CLIPPromptEncoder:
    """texts -> (pooled [B, 1, D], mask) in the calling convention of the other prompt encoders;
    ``encode`` gives all three outputs."""

    def __init__(self, model: CLIPTextEncoder, tokenizer, max_len: int = 77):
        self.model, self.tokenizer, self.max_len = model, tokenizer, max_len

    @classmethod
    def from_pretrained(cls, model_path: str, subfolder: str, tokenizer_subfolder: str, dtype, device, with_projection=None):
        from transformers import AutoTokenizer
        with open(os.path.join(model_path, subfolder, "config.json")) as f:
            d = json.load(f)
        if with_projection:
            d["_with_projection"] = True
        cfg = CLIPTextConfig.from_dict(d)
        tok = AutoTokenizer.from_pretrained(os.path.join(model_path, tokenizer_subfolder))
        return cls(CLIPTextEncoder(cfg, dtype, device), tok, min(77, cfg.max_position_embeddings))

    def load_weights(self, weights) -> set:
        return self.model.load_weights(weights)

    @torch.no_grad()
    def encode(self, texts, device):
        enc = self.tokenizer(list(texts), padding="max_length", max_length=self.max_len, truncation=True, return_tensors="pt")
        return self.model(enc["input_ids"].to(device))

    def __call__(self, texts, device, dtype=None, max_len=None):
        _, pooled, _ = self.encode(texts, device)
        pooled = pooled[:, None]
        return (pooled if dtype is None else pooled.to(dtype)), torch.ones(pooled.shape[:2], dtype=torch.long, device=pooled.device)
