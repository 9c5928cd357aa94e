"""Qwen2.5-Omni thinker: dense Qwen2.5 decoder with MRoPE, audio and vision towers.  Besides text
it emits the final hidden state of every prompt and generated token ("latent"), which the talker
is conditioned on (vllm_omni/model_executor/models/qwen2_5_omni/qwen2_5_omni.py:199-366)."""
from __future__ import annotations

import torch

from ..qwen3_omni.thinker import Qwen3OmniMoeThinker
from ..qwen_decoder import QwenDecoderModel
from ..qwen2_5_vl_vision import Qwen25VisionTower
from .audio import Qwen25AudioEncoder
from ..base import StageModel
from .config import Qwen25OmniConfig


class Qwen25OmniThinker(Qwen3OmniMoeThinker):
    """Shares the multimodal preprocessing (placeholder expansion, MRoPE ids) with the Qwen3 thinker;
    differs in the decoder (dense, qkv bias, no q/k norm) and in what it hands on."""
    engine_output_type = "latent"

    def __init__(self, cfg: Qwen25OmniConfig, dtype=torch.bfloat16, device=None):
        StageModel.__init__(self, cfg.thinker, dtype, device)
        self.cfg = cfg
        self.decoder = QwenDecoderModel(cfg.thinker, dtype, device)
        self.audio_tower = Qwen25AudioEncoder(cfg.audio, dtype, device)
        self.visual = Qwen25VisionTower(cfg.vision, dtype, device)      # window-attention ViT of Qwen2.5-VL
        self.capture = (0,)

    def forward_batch(self, batch, kv_caches, sched):
        return self.decoder(batch, kv_caches, capture_layers=self.capture)

    def collect_outputs(self, sched, batch, hidden, captured) -> None:
        """Per token the talker gets (final hidden state + input embedding); the embeddings of audio /
        image / video placeholder rows count as zero (transformers' Qwen2.5-Omni ``generate``)."""
        cfg = self.cfg
        emb = captured[0]
        ids = batch.input_ids
        mm = (ids == cfg.audio_token_id) | (ids == cfg.image_token_id) | (ids == cfg.video_token_id)
        state = hidden + torch.where(mm[:, None], torch.zeros_like(emb), emb)
        row = 0
        for s in sched.scheduled:
            n = s.num_new_tokens
            r = s.request
            r.multimodal_outputs.setdefault("latent", []).append(state[row:row + n])
            if "tts_bos_embed" not in r.multimodal_outputs:
                e = self.decoder.embed_tokens
                for key, tid in (("tts_bos_embed", cfg.tts_text_bos_id), ("tts_eos_embed", cfg.tts_text_eos_id),
                                 ("tts_pad_embed", cfg.tts_text_pad_id)):
                    r.multimodal_outputs[key] = [e[tid % e.shape[0]][None]]
            row += n
