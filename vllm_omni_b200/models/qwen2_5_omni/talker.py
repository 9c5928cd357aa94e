"""Qwen2.5-Omni talker: a small dense decoder over codec tokens, conditioned on the thinker's
hidden states through one projection (vllm_omni/model_executor/models/qwen2_5_omni/
qwen2_5_omni.py:642-795).

Parametrisation of the checkpoint: the codec embedding table lives in the THINKER width
(``talker.model.embed_tokens`` [vocab, embedding_size]); every input row is (codec embedding +
thinker state) in that width and goes through ``thinker_to_talker_proj`` into the talker width.

Inputs as in transformers' ``generate`` (thinker state = final hidden + token embedding):
prefill rows = [prompt states..., embedding of the tts text-bos token, first reply state], with the
codec PAD embedding added to the second-to-last and the codec BOS embedding to the last row; decode
step k feeds embedding(codec token k-1) + r[k] with r = [reply states 1.., text-eos embedding,
text-pad embedding], staying on the last entry once the reply is used up.  The codec BOS id is
never sampled; sampling stops at the codec EOS id."""
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
        import dataclasses
        # the decoder never looks tokens up itself: all rows arrive as projected embeddings
        self.decoder = QwenDecoderModel(dataclasses.replace(cfg.talker, vocab_size=8), dtype, device, with_lm_head=False)
        E = cfg.talker_embedding_size
        self.codec_embedding = torch.nn.Parameter(torch.empty(cfg.talker.vocab_size, E, dtype=dtype, device=device)
                                                  .normal_(0, 0.02), requires_grad=False)
        self.thinker_to_talker_proj = FusedLinear(E, cfg.talker.hidden_size, bias=True, dtype=dtype, device=device)
        self.codec_head = FusedLinear(cfg.talker.hidden_size, cfg.talker.vocab_size, bias=False, dtype=dtype,
                                      device=device)

    def eos_token_id(self):
        return self.cfg.codec_eos_id

    @torch.no_grad()
    def preprocess_request(self, req) -> None:
        info = req.additional_information
        if "prompt_embeds" not in info:
            return
        cfg, dev = self.cfg, self.codec_embedding.device
        codec = self.codec_embedding
        V = codec.shape[0]
        prompt = info["prompt_embeds"].to(dev, self.dtype_)
        reply = info["thinker_result"].to(dev, self.dtype_)
        zero = prompt.new_zeros(1, prompt.shape[1])
        special = lambda k: info[k].to(dev, self.dtype_).reshape(1, -1) if k in info else zero
        first = reply[:1] if reply.shape[0] else zero
        head = torch.cat([prompt, special("tts_bos_embed"), first], 0)
        head[-2] += codec[cfg.codec_pad_id % V]
        head[-1] += codec[cfg.codec_bos_id % V]
        head = self.thinker_to_talker_proj(head.contiguous())
        req.prompt_embeds = head
        req.prompt_token_ids = [0] * head.shape[0]
        steps = torch.cat([reply[1:], special("tts_eos_embed"), special("tts_pad_embed")], 0)
        req.runtime_state.update(reply=steps, next_embed=None)

    def input_embeds_for(self, req, start, n):
        if start < req.num_prompt_tokens:
            return req.prompt_embeds[start:start + n]
        return req.runtime_state.get("next_embed")

    def compute_logits(self, hidden):
        logits = self.codec_head(hidden)
        logits[..., self.cfg.codec_bos_id % logits.shape[-1]] = float("-inf")      # the start marker is never spoken
        return logits

    @torch.no_grad()
    def postprocess_sampled(self, reqs, ids, hidden):
        codec = self.codec_embedding
        tok = ids.long().clamp(0, codec.shape[0] - 1)
        emb = codec[tok]
        for i, r in enumerate(reqs):
            st = r.runtime_state
            k = len(r.output_token_ids)                       # index of the codec token just sampled
            reply = st.get("reply")
            nxt = emb[i:i + 1]
            if reply is not None and reply.shape[0]:
                j = min(k, reply.shape[0] - 1)
                nxt = nxt + reply[j:j + 1]
            st["next_embed"] = self.thinker_to_talker_proj(nxt.contiguous())
            r.multimodal_outputs.setdefault("codes", []).append(tok[i:i + 1, None])
        return ids

    @torch.no_grad()
    def load_weights(self, weights):
        """Checkpoint names under ``talker.``: ``model.embed_tokens`` (codec table, thinker width),
        ``model.layers.* / model.norm``, ``thinker_to_talker_proj.*``, ``codec_head.weight``."""
        dec, loaded = [], set()
        direct = {"model.embed_tokens.weight": self.codec_embedding, "codec_head.weight": self.codec_head.weight,
                  "thinker_to_talker_proj.weight": self.thinker_to_talker_proj.weight,
                  "thinker_to_talker_proj.bias": self.thinker_to_talker_proj.bias}
        for full, w in weights:
            if full.startswith(("thinker.", "token2wav.")):
                continue
            n = full[len("talker."):] if full.startswith("talker.") else full
            if n in direct:
                direct[n].copy_(w.to(direct[n].dtype))
                loaded.add(full)
            else:
                dec.append((n, w, full))
        names = {n: full for n, _, full in dec}
        return loaded | {names[n] for n in self.decoder.load_weights([(n, w) for n, w, _ in dec])}
