"""Prompt encoder of FLUX.2-klein: a Qwen3 causal LM over the chat-templated prompt, padded to the
full text length; the hidden states entering layers 9, 18 and 27 are laid side by side per token, so
the conditioning width is three times the LM width
(vllm_omni/diffusion/models/flux2_klein/pipeline_flux2_klein.py:247-303).

The padded positions are part of the conditioning: the DiT attends to all 512 rows.  Their states
follow transformers' masking rule — a padded query sees the real tokens before it but no padded key —
so the encoder runs a dense masked pass over this framework's decoder weights (once per request)
instead of the packed causal path that skips padding.
"""
from __future__ import annotations

import json
import os

import torch
import torch.nn.functional as F

from ....models.qwen_decoder import DecoderConfig, QwenDecoderModel
from ....ops import fused


@torch.no_grad()
def dense_hidden_states(model: QwenDecoderModel, ids: torch.Tensor, mask: torch.Tensor, layers) -> list[torch.Tensor]:
    """ids, mask [B, L] -> the states entering each layer of ``layers`` ([B, L, D] each).  Attention is
    causal over positions 0..L-1 and never reads a key whose mask is 0."""
    cfg = model.cfg
    H, Hkv, Dh, eps = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps
    B, L = ids.shape
    dev = ids.device
    x = model.embed_tokens[ids]
    cos, sin = model.rope.cos_sin_for(torch.arange(L, device=dev))
    i = torch.arange(L, device=dev)
    allow = (i[None, :] <= i[:, None])[None] & mask.bool()[:, None, :]                 # [B, Lq, Lk]
    bias = torch.zeros(B, 1, L, L, dtype=torch.float32, device=dev).masked_fill_(~allow[:, None], torch.finfo(torch.float32).min)
    want, out = set(int(k) for k in layers), {}
    for li, layer in enumerate(model.layers):
        if li in want:
            out[li] = x
        if li >= max(want):
            break
        h = fused.norm_modulate(x, weight=layer.input_layernorm, rms=True, eps=eps)
        qkv = layer.qkv_proj(h).view(B, L, -1)
        if qkv.is_cuda and Dh not in (64, 128):
            qkv = fused.qk_norm_rope_reference(qkv, H, Hkv, Dh, layer.q_norm, layer.k_norm, None, None, 1 << 30, cos, sin, False, eps)
        else:
            fused.qk_norm_rope_(qkv, H, Hkv, Dh, wq=layer.q_norm, wk=layer.k_norm, cos=cos, sin=sin, interleaved=False, eps=eps)
        q = qkv[..., :H * Dh].view(B, L, H, Dh).transpose(1, 2)
        k = qkv[..., H * Dh:(H + Hkv) * Dh].view(B, L, Hkv, Dh).transpose(1, 2)
        v = qkv[..., (H + Hkv) * Dh:].view(B, L, Hkv, Dh).transpose(1, 2)
        if Hkv != H:
            k, v = k.repeat_interleave(H // Hkv, dim=1), v.repeat_interleave(H // Hkv, dim=1)
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=bias.to(q.dtype)).transpose(1, 2).reshape(B, L, H * Dh)
        x = layer.o_proj(o.contiguous(), residual=x)
        h = fused.norm_modulate(x, weight=layer.post_attention_layernorm, rms=True, eps=eps)
        x = layer.down(fused.silu_mul(layer.gate_up(h)), residual=x)
    return [out[int(k)] for k in layers]


class Flux2PromptEncoder:
    def __init__(self, cfg: DecoderConfig, tokenizer, dtype=torch.bfloat16, device=None, max_length: int = 512,
                 layers=(9, 18, 27)):
        self.cfg, self.tokenizer, self.max_length, self.layers = cfg, tokenizer, max_length, tuple(layers)
        self.model = QwenDecoderModel(cfg, dtype, device, with_lm_head=False)

    @classmethod
    def from_pretrained(cls, model_path: str, dtype=torch.bfloat16, device=None, **kw) -> "Flux2PromptEncoder":
        from transformers import AutoTokenizer
        with open(os.path.join(model_path, "text_encoder", "config.json")) as f:
            cfg = DecoderConfig.from_dict(json.load(f))
        return cls(cfg, AutoTokenizer.from_pretrained(os.path.join(model_path, "tokenizer")), dtype, device, **kw)

    def _text(self, prompt: str) -> str:
        msgs = [{"role": "user", "content": prompt}]
        try:
            return self.tokenizer.apply_chat_template(msgs, tokenize=False, add_generation_prompt=True, enable_thinking=False)
        except TypeError:
            return self.tokenizer.apply_chat_template(msgs, tokenize=False, add_generation_prompt=True)

    @torch.no_grad()
    def __call__(self, prompts, device=None, dtype=None, max_sequence_length: int | None = None, layers=None):
        """Returns (states [B, L, len(layers) * D], all-ones mask [B, L]); L = the padded text length."""
        dev = self.model.embed_tokens.device
        L = min(int(max_sequence_length or self.max_length), self.max_length)
        enc = self.tokenizer([self._text(p) for p in prompts], return_tensors="pt", padding="max_length", truncation=True,
                             max_length=L)
        ids, mask = enc["input_ids"].to(dev), enc["attention_mask"].to(dev)
        states = dense_hidden_states(self.model, ids, mask, layers or self.layers)
        out = torch.stack(states, dim=2).reshape(ids.shape[0], L, -1)           # per token: [layer a | layer b | layer c]
        out = out.to(device=device or dev, dtype=dtype or out.dtype)
        return out, torch.ones(out.shape[:2], dtype=torch.long, device=out.device)

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        return self.model.load_weights([(n, w) for n, w in weights if not n.startswith("lm_head.")])
