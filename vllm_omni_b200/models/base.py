"""Interface between the AR engine's model runner and a stage model, with the behaviour of a
plain text decoder as the default.  Omni stage models (thinker, talker, code2wav ...) override
the hooks: per-request prompt-embedding overlays and preprocessing
(vllm_omni/worker/gpu_model_runner.py:764-1083), hidden-state capture, extra sampling steps."""
from __future__ import annotations

import torch
from torch import nn

from .qwen_decoder import DecoderConfig, ModelBatch, QwenDecoderModel


class StageModel(nn.Module):
    engine_output_type = "text"         # text | latent | audio
    is_generation_model = False         # True: one-shot (non-autoregressive) stage

    def __init__(self, decoder_config: DecoderConfig | None, dtype, device):
        super().__init__()
        self.decoder_config = decoder_config
        self.dtype_, self.device_ = dtype, device

    # ---- inputs
    def positions_for(self, req, start: int, n: int) -> torch.Tensor:
        mp = req.runtime_state.get("mrope_positions")
        if mp is not None:                       # [3, L] for the prompt; text continues linearly
            L = mp.shape[1]
            cols = []
            for t in range(start, start + n):
                cols.append(mp[:, t] if t < L else (mp[:, -1].max() + 1 + (t - L)).expand(3))
            return torch.stack(cols, dim=1)
        return torch.arange(start, start + n)

    def input_embeds_for(self, req, start: int, n: int):
        pe = req.prompt_embeds
        if pe is None or start >= pe.shape[0]:
            return None
        e = pe[start:start + n]
        if e.shape[0] < n:          # the tail (generated tokens) uses the embedding table
            return None if e.shape[0] == 0 else e
        return e

    # ---- forward
    def forward_batch(self, batch: ModelBatch, kv_caches, sched):
        return self.decoder(batch, kv_caches)

    def compute_logits(self, hidden):
        return self.decoder.compute_logits(hidden)

    def postprocess_sampled(self, reqs, ids, hidden):
        return ids

    def collect_outputs(self, sched, batch, hidden, captured) -> None:
        pass

    def generate_for(self, req, start, n):
        raise NotImplementedError

    def eos_token_id(self):
        return None


class TextDecoderModel(StageModel):
    """A plain causal LM stage."""

    def __init__(self, cfg: DecoderConfig, dtype=torch.bfloat16, device=None):
        super().__init__(cfg, dtype, device)
        self.decoder = QwenDecoderModel(cfg, dtype, device)

    def load_weights(self, weights):
        pre = "language_model."                          # multimodal checkpoints nest the LM under this prefix
        strip = lambda n: n[len(pre):] if n.startswith(pre) else n
        loaded = self.decoder.load_weights((strip(n), w) for n, w in weights)
        return loaded
