"""Qwen2.5-Omni thinker: dense Qwen2.5 decoder with MRoPE, audio and vision towers.  Besides text
it emits the final hidden state of every prompt and generated token ("latent"), which the talker
is conditioned on (vllm_omni/model_executor/models/qwen2_5_omni/qwen2_5_omni.py:199-366)."""
from __future__ import annotations

import torch

from ..qwen3_omni.thinker import Qwen3OmniMoeThinker
from ..qwen_decoder import QwenDecoderModel
from ..qwen2_5_vl_vision import Qwen25VisionTower
from ..qwen3_omni.encoders import AudioEncoder
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
        self.audio_tower = AudioEncoder(cfg.audio, dtype, device)
        self.visual = Qwen25VisionTower(cfg.vision, dtype, device)      # window-attention ViT of Qwen2.5-VL
        self.capture = ()

    def forward_batch(self, batch, kv_caches, sched):
        return self.decoder(batch, kv_caches)

    def collect_outputs(self, sched, batch, hidden, captured) -> None:
        row = 0
        for s in sched.scheduled:
            n = s.num_new_tokens
            s.request.multimodal_outputs.setdefault("latent", []).append(hidden[row:row + n])
            row += n
