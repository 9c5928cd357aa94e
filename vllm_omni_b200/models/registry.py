"""AR / generation model registry: ``model_arch`` (+ ``model_stage``) -> stage model class
(vllm_omni/model_executor/models/registry.py)."""
from __future__ import annotations

import importlib

_MODELS: dict[str, tuple[str, str]] = {
    "Qwen3OmniMoeForConditionalGeneration": ("vllm_omni_b200.models.qwen3_omni.model", "build_qwen3_omni_stage"),
    "Qwen2_5OmniForConditionalGeneration": ("vllm_omni_b200.models.qwen2_5_omni.model", "build_qwen2_5_omni_stage"),
    "Qwen3TTSForConditionalGeneration": ("vllm_omni_b200.models.qwen3_tts.model", "build_qwen3_tts_stage"),
    "Qwen3ForCausalLM": ("vllm_omni_b200.models.text", "build_text_model"),
    "Qwen2ForCausalLM": ("vllm_omni_b200.models.text", "build_text_model"),
    "Qwen3MoeForCausalLM": ("vllm_omni_b200.models.text", "build_text_model"),
    "BagelForConditionalGeneration": ("vllm_omni_b200.models.text", "build_text_model"),
}


def register_model(arch: str, module: str, factory: str) -> None:
    _MODELS[arch] = (module, factory)


def supported_archs() -> list[str]:
    return sorted(_MODELS)


def build_stage_model(model_arch: str, model_stage: str | None, hf_config: dict, dtype, device, **kw):
    if model_arch not in _MODELS:
        raise ValueError(f"unknown model_arch {model_arch!r}; supported: {supported_archs()}")
    mod, fn = _MODELS[model_arch]
    return getattr(importlib.import_module(mod), fn)(model_stage, hf_config, dtype, device, **kw)
