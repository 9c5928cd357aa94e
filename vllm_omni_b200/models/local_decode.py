"""Private autoregressive loop for models that generate INSIDE one stage step (Qwen3-TTS, the
code predictors): a ``QwenDecoderModel`` driven over its own small paged KV cache, so that it
runs on the same paged-attention kernels as the engine's stages without going through the
scheduler.  The reference runs such inner loops with HF ``generate``-style code and no KV
cache or CUDA-graph buffers (vllm_omni/model_executor/models/qwen3_omni/
qwen3_omni_moe_code_predictor_mtp.py:413-524, qwen3_tts/modeling_qwen3_tts.py).
"""
from __future__ import annotations

import torch

from .qwen_decoder import ModelBatch, PrefillSeg, QwenDecoderModel


class LocalDecodeSession:
    """One sequence: ``prefill(embeds)`` then ``step(embed)`` repeatedly.  Positions are linear."""

    def __init__(self, decoder: QwenDecoderModel, max_len: int, block_size: int = 16):
        cfg = decoder.cfg
        self.decoder, self.bs = decoder, block_size
        dev = decoder.embed_tokens.device
        dtype = decoder.embed_tokens.dtype
        nb = (max_len + block_size - 1) // block_size
        self.max_len = nb * block_size
        # zero-initialised pools: partially filled pages are read (and masked) by the attention kernel
        self.caches = [(torch.zeros(nb, block_size, cfg.num_key_value_heads, cfg.head_dim, dtype=dtype, device=dev),
                        torch.zeros(nb, block_size, cfg.num_key_value_heads, cfg.head_dim, dtype=dtype, device=dev))
                       for _ in range(cfg.num_hidden_layers)]
        self.table = torch.arange(nb, dtype=torch.int32, device=dev)
        self.len = 0
        self.dev = dev

    def reset(self):
        self.len = 0

    def _batch(self, n, embeds, ids):
        dev = self.dev
        if self.len + n > self.max_len:
            raise ValueError(f"local decode session is full ({self.max_len} tokens)")
        pos = torch.arange(self.len, self.len + n, device=dev)
        slots = pos.to(torch.int32)                         # page i holds tokens [i*bs, (i+1)*bs)
        if ids is None:
            ids = torch.zeros(n, dtype=torch.long, device=dev)
        kw = {}
        if embeds is not None:
            kw = dict(input_embeds=embeds.to(dev), embeds_mask=torch.ones(n, dtype=torch.bool, device=dev))
        return pos, slots, ids, kw

    @torch.no_grad()
    def prefill(self, embeds: torch.Tensor | None = None, ids: torch.Tensor | None = None, capture_layers=()):
        n = embeds.shape[0] if embeds is not None else ids.shape[0]
        pos, slots, ids, kw = self._batch(n, embeds, ids)
        b = ModelBatch(ids.to(self.dev), pos, slots, [PrefillSeg(0, n, self.len, self.table)], **kw)
        hidden, cap = self.decoder(b, self.caches, capture_layers=capture_layers)
        self.len += n
        return (hidden, cap) if capture_layers else hidden

    @torch.no_grad()
    def step(self, embed: torch.Tensor | None = None, token: int | None = None):
        """Append one token (by embedding row [1, D] or by id); returns its final hidden state [1, D]."""
        ids = None if token is None else torch.tensor([token], dtype=torch.long, device=self.dev)
        pos, slots, ids, kw = self._batch(1, embed, ids)
        b = ModelBatch(ids, pos, slots, [], decode_rows=torch.zeros(1, dtype=torch.long, device=self.dev),
                       decode_block_tables=self.table[None].contiguous(),
                       decode_seq_lens=torch.tensor([self.len + 1], dtype=torch.int32, device=self.dev), **kw)
        hidden, _ = self.decoder(b, self.caches)
        self.len += 1
        return hidden
