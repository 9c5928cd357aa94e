"""Qwen2.5-VL language model as the Qwen-Image prompt encoder.

The reference pipeline wraps each prompt in a fixed ChatML template, runs the Hugging Face
``Qwen2_5_VLForConditionalGeneration`` and keeps the last hidden states (after the final norm) of
the tokens that follow the 34-token template head, zero padded per batch with a mask
(vllm_omni/diffusion/models/qwen_image/pipeline_qwen_image.py:292-405).  Here the language model
is this framework's decoder (same kernels as the AR stages): all prompts of a call are packed
into one flat batch of causal prefill segments, so no padding is computed.  For text-only input
the three MRoPE axes carry the same index, i.e. plain rotary positions.

Checkpoint names: ``text_encoder.model.language_model.*`` (or the older ``text_encoder.model.*``);
the vision tower's tensors (``visual.*``) are not needed for text-to-image and are skipped.
"""
from __future__ import annotations

import json
import os

import torch

from ....models.qwen_decoder import DecoderConfig, ModelBatch, PrefillSeg, QwenDecoderModel

PROMPT_TEMPLATE = ("<|im_start|>system\nDescribe the image by detailing the color, shape, size, texture, quantity, text, "
                   "spatial relationships of the objects and background:<|im_end|>\n<|im_start|>user\n{}<|im_end|>\n"
                   "<|im_start|>assistant\n")
TEMPLATE_DROP_TOKENS = 34
TOKENIZER_MAX_LENGTH = 1024


def text_config_from_hf(d: dict) -> DecoderConfig:
    """Qwen2.5-VL config.json (flat, or with a ``text_config`` sub-dict) -> decoder geometry."""
    t = dict(d.get("text_config") or d)
    t.setdefault("attention_bias", True)          # Qwen2 family: biases on q/k/v, no q/k norm
    t["qk_norm"] = False
    cfg = DecoderConfig.from_dict(t)
    cfg.mrope_section = None                      # text-only: the three axes coincide
    return cfg


class QwenVLTextEncoder:
    def __init__(self, cfg: DecoderConfig, tokenizer, dtype=torch.bfloat16, device=None,
                 template: str = PROMPT_TEMPLATE, drop_tokens: int = TEMPLATE_DROP_TOKENS):
        self.cfg, self.tokenizer = cfg, tokenizer
        self.model = QwenDecoderModel(cfg, dtype, device, with_lm_head=False)
        self.template, self.drop = template, drop_tokens

    @classmethod
    def from_pretrained(cls, model_path: str, dtype=torch.bfloat16, device=None, **kw) -> "QwenVLTextEncoder":
        """``model_path``: a diffusers pipeline directory with ``text_encoder/`` and ``tokenizer/``."""
        from ....engine.tokenizer import get_tokenizer
        with open(os.path.join(model_path, "text_encoder", "config.json")) as f:
            cfg = text_config_from_hf(json.load(f))
        return cls(cfg, get_tokenizer(os.path.join(model_path, "tokenizer")), dtype, device, **kw)

    def to(self, *a, **k):
        self.model.to(*a, **k)
        return self

    @torch.no_grad()
    def __call__(self, prompts: list[str], device=None, dtype=None, max_sequence_length: int | None = None):
        """Returns (states [B, L, D] zero padded, mask [B, L] int64)."""
        dev = self.model.embed_tokens.device
        seqs = []
        for p in prompts:
            ids = self.tokenizer.encode(self.template.format(p), add_special_tokens=False)
            seqs.append(list(ids)[:TOKENIZER_MAX_LENGTH + self.drop])
        flat = torch.tensor([t for s in seqs for t in s], dtype=torch.long, device=dev)
        pos = torch.cat([torch.arange(len(s), device=dev) for s in seqs])
        segs, row = [], 0
        for s in seqs:
            segs.append(PrefillSeg(row, len(s), 0, None))
            row += len(s)
        batch = ModelBatch(flat, pos, torch.full((row,), -1, dtype=torch.int32, device=dev), segs)
        hidden, _ = self.model(batch, None)
        outs, row = [], 0
        for s in seqs:
            outs.append(hidden[row + self.drop:row + len(s)])
            row += len(s)
        L = max(1, max(o.shape[0] for o in outs))
        if max_sequence_length:
            L = min(L, max_sequence_length)
        states = hidden.new_zeros(len(seqs), L, hidden.shape[-1])
        mask = torch.zeros(len(seqs), L, dtype=torch.long, device=dev)
        for i, o in enumerate(outs):
            n = min(L, o.shape[0])
            states[i, :n] = o[:n]
            mask[i, :n] = 1
        return states.to(device=device or dev, dtype=dtype or states.dtype), mask.to(device or dev)

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        """Names relative to ``text_encoder.``."""
        mapped, back = [], {}
        for n, w in weights:
            if "visual." in n or n.startswith("lm_head."):
                continue
            m = n.replace("model.language_model.", "model.", 1) if n.startswith("model.language_model.") else n
            mapped.append((m, w))
            back[m] = n
        return {back[m] for m in self.model.load_weights(mapped)}
