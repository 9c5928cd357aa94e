"""Qwen2.5-Omni talker: a small dense decoder over codec tokens, conditioned on the thinker's
hidden states through one projection (vllm_omni/model_executor/models/qwen2_5_omni/
qwen2_5_omni.py:642-795).

Prompt rows: projection of the thinker's prompt hidden states plus the codec PAD embedding, then one
row for the first generated text token plus the codec BOS embedding.  Decode step k feeds the
embedding of codec token k-1 plus the projected hidden state of generated text token k (until the
thinker's reply is used up).  Sampling stops at the codec EOS id."""
from __future__ import annotations

import torch

from ...diffusion.layers.linear import FusedLinear
from ..base import StageModel
from ..qwen_decoder import QwenDecoderModel
from .config import Qwen25OmniConfig


class Qwen25OmniTalker(StageModel):
    engine_output_type = "latent"
    stream_output_keys = ("codes",)

    def __init__(self, cfg: Qwen25OmniConfig, dtype=torch.bfloat16, device=None):
        super().__init__(cfg.talker, dtype, device)
        self.cfg = cfg
        self.decoder = QwenDecoderModel(cfg.talker, dtype, device, with_lm_head=False)
        self.thinker_to_talker_proj = FusedLinear(cfg.thinker.hidden_size, cfg.talker.hidden_size, bias=True,
                                                  dtype=dtype, device=device)
        self.codec_head = FusedLinear(cfg.talker.hidden_size, cfg.talker.vocab_size, bias=False, dtype=dtype,
                                      device=device)

    def eos_token_id(self):
        return self.cfg.codec_eos_id

    @torch.no_grad()
    def preprocess_request(self, req) -> None:
        info = req.additional_information
        if "prompt_embeds" not in info:
            return
        cfg, dev = self.cfg, self.decoder.embed_tokens.device
        codec = self.decoder.embed_tokens
        V = codec.shape[0]
        prompt = self.thinker_to_talker_proj(info["prompt_embeds"].to(dev, self.dtype_).contiguous())
        reply = info["thinker_result"].to(dev, self.dtype_)
        reply = self.thinker_to_talker_proj(reply.contiguous()) if reply.shape[0] else prompt.new_zeros(0, prompt.shape[1])
        first = reply[:1] if reply.shape[0] else prompt.new_zeros(1, prompt.shape[1])
        head = torch.cat([prompt + codec[cfg.codec_pad_id % V][None], first + codec[cfg.codec_bos_id % V][None]], 0)
        req.prompt_embeds = head
        req.prompt_token_ids = [0] * head.shape[0]
        req.runtime_state.update(reply=reply, next_embed=None)

    def input_embeds_for(self, req, start, n):
        if start < req.num_prompt_tokens:
            return req.prompt_embeds[start:start + n]
        return req.runtime_state.get("next_embed")

    def compute_logits(self, hidden):
        return self.codec_head(hidden)

    @torch.no_grad()
    def postprocess_sampled(self, reqs, ids, hidden):
        codec = self.decoder.embed_tokens
        tok = ids.long().clamp(0, codec.shape[0] - 1)
        emb = codec[tok]
        for i, r in enumerate(reqs):
            st = r.runtime_state
            k = len(r.output_token_ids) + 1                   # text row that conditions the NEXT codec token
            reply = st.get("reply")
            nxt = emb[i:i + 1]
            if reply is not None and k < reply.shape[0]:
                nxt = nxt + reply[k:k + 1]
            st["next_embed"] = nxt
            r.multimodal_outputs.setdefault("codes", []).append(tok[i:i + 1, None])
        return ids

    def load_weights(self, weights):
        ws = [(n[len("talker."):] if n.startswith("talker.") else n, w) for n, w in weights]
        return self.decoder.load_weights(ws)
