"""Plain causal-LM stages (Qwen2 / Qwen3 / Qwen3-MoE text models)."""
from __future__ import annotations

from .base import TextDecoderModel
from .qwen_decoder import DecoderConfig


def build_text_model(model_stage, hf_config: dict, dtype, device, **kw):
    cfg = hf_config.get("text_config", hf_config)
    dc = DecoderConfig.from_dict(cfg) if cfg else DecoderConfig()
    if "num_experts" not in cfg:
        dc.num_experts = 0
    if kw.get("tiny"):
        dc = DecoderConfig(vocab_size=259, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                           num_key_value_heads=2, head_dim=16, intermediate_size=128)
    return TextDecoderModel(dc, dtype, device)
