"""Caption encoder of the Z-Image pipeline: a Qwen3 causal LM whose second-to-last hidden layer
(before the final norm) over the chat-templated prompt conditions the DiT
(vllm_omni/diffusion/models/z_image/pipeline_z_image.py:236-270).  Runs on this framework's decoder;
prompts are packed into one batch of causal segments, so nothing is computed for padding."""
from __future__ import annotations

import json
import os

import torch

from ....models.qwen_decoder import DecoderConfig, ModelBatch, PrefillSeg, QwenDecoderModel


class QwenCaptionEncoder:
    def __init__(self, cfg: DecoderConfig, tokenizer, dtype=torch.bfloat16, device=None, max_length: int = 512):
        self.cfg, self.tokenizer, self.max_length = cfg, tokenizer, max_length
        self.model = QwenDecoderModel(cfg, dtype, device, with_lm_head=False)

    @classmethod
    def from_pretrained(cls, model_path: str, dtype=torch.bfloat16, device=None, **kw) -> "QwenCaptionEncoder":
        from ....engine.tokenizer import get_tokenizer
        with open(os.path.join(model_path, "text_encoder", "config.json")) as f:
            cfg = DecoderConfig.from_dict(json.load(f))
        return cls(cfg, get_tokenizer(os.path.join(model_path, "tokenizer")), dtype, device, **kw)

    def _ids(self, prompt: str) -> list[int]:
        msgs = [{"role": "user", "content": prompt}]
        try:
            text = self.tokenizer.apply_chat_template(msgs, tokenize=False, add_generation_prompt=True, enable_thinking=True)
        except TypeError:
            text = self.tokenizer.apply_chat_template(msgs, tokenize=False, add_generation_prompt=True)
        return list(self.tokenizer.encode(text, add_special_tokens=False))

    @torch.no_grad()
    def __call__(self, prompts: list[str], device=None, dtype=None, max_sequence_length: int | None = None):
        """Returns (states [B, L, D] zero padded, mask [B, L])."""
        dev = self.model.embed_tokens.device
        limit = min(max_sequence_length or self.max_length, self.max_length)
        seqs = [self._ids(p)[:limit] for p in prompts]
        flat = torch.tensor([t for s in seqs for t in s], dtype=torch.long, device=dev)
        pos = torch.cat([torch.arange(len(s), device=dev) for s in seqs])
        segs, row = [], 0
        for s in seqs:
            segs.append(PrefillSeg(row, len(s), 0, None))
            row += len(s)
        n = self.cfg.num_hidden_layers
        batch = ModelBatch(flat, pos, torch.full((row,), -1, dtype=torch.int32, device=dev), segs)
        _, cap = self.model(batch, None, capture_layers=(n - 1,))       # output of layer n-2 = hidden_states[-2]
        hidden = cap[n - 1]
        L = max(len(s) for s in seqs)
        states = hidden.new_zeros(len(seqs), L, hidden.shape[-1])
        mask = torch.zeros(len(seqs), L, dtype=torch.long, device=dev)
        row = 0
        for i, s in enumerate(seqs):
            states[i, :len(s)] = hidden[row:row + len(s)]
            mask[i, :len(s)] = 1
            row += len(s)
        return states.to(device=device or dev, dtype=dtype or states.dtype), mask.to(device or dev)

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        return self.model.load_weights([(n, w) for n, w in weights if not n.startswith("lm_head.")])
