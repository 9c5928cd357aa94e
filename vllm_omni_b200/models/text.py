"""Plain causal-LM stages (Qwen2 / Qwen3 / Qwen3-MoE text models) and the understanding half of BAGEL:
its checkpoint nests a Qwen2 config with per-head q/k norms under ``llm_config`` and names the weights
``language_model.model.*`` (the ``*_moe_gen`` twins belong to the image-generation stage and are skipped)."""
from __future__ import annotations

from .base import TextDecoderModel
from .qwen_decoder import DecoderConfig


def build_text_model(model_stage, hf_config: dict, dtype, device, **kw):
    cfg = hf_config.get("text_config", hf_config)
    if hf_config.get("llm_config"):                       # BAGEL
        cfg = dict(hf_config["llm_config"])
        cfg.setdefault("qk_norm", True)
        cfg.setdefault("attention_bias", True)
    dc = DecoderConfig.from_dict(cfg) if cfg else DecoderConfig()
    if "num_experts" not in cfg:
        dc.num_experts = 0
    if kw.get("tiny"):
        # test geometry; ``moe`` / ``head_dim`` choose the mixture-of-experts layers and the head size
        dc = DecoderConfig(vocab_size=int(kw.get("vocab_size", 259)), hidden_size=64, num_hidden_layers=2,
                           num_attention_heads=4, num_key_value_heads=2, head_dim=int(kw.get("head_dim", 16)),
                           intermediate_size=128, num_experts=8 if kw.get("moe") else 0, num_experts_per_tok=2,
                           moe_intermediate_size=64)
    return TextDecoderModel(dc, dtype, device)
