"""``Qwen2_5OmniForConditionalGeneration``: one architecture name, three stage models chosen by
``model_stage`` (thinker | talker | code2wav), as in the reference's unified class
(vllm_omni/model_executor/models/qwen2_5_omni/qwen2_5_omni.py:55-140)."""
from __future__ import annotations

from .config import Qwen25OmniConfig
from .talker import Qwen25OmniTalker
from .thinker import Qwen25OmniThinker
from .token2wav import Qwen25OmniToken2Wav


def build_qwen2_5_omni_stage(model_stage, hf_config: dict, dtype, device, **kw):
    if kw.get("tiny") or (hf_config or {}).get("tiny"):
        cfg = Qwen25OmniConfig.tiny()
    elif hf_config:
        cfg = Qwen25OmniConfig.from_hf(hf_config)
    else:
        cfg = Qwen25OmniConfig()
    stage = (model_stage or "thinker").lower()
    if stage == "thinker":
        return Qwen25OmniThinker(cfg, dtype, device)
    if stage == "talker":
        return Qwen25OmniTalker(cfg, dtype, device)
    if stage in ("code2wav", "token2wav"):
        return Qwen25OmniToken2Wav(cfg, dtype, device)
    raise ValueError(f"unknown model_stage {model_stage!r} for Qwen2.5-Omni")
