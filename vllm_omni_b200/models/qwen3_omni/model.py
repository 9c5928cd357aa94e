"""``Qwen3OmniMoeForConditionalGeneration``: one architecture name, three stage models chosen
by ``model_stage`` (thinker | talker | code2wav), like the reference's unified class
(vllm_omni/model_executor/models/qwen3_omni/qwen3_omni.py:71-1158)."""
from __future__ import annotations

from .code2wav import Qwen3OmniCode2Wav
from .config import Qwen3OmniConfig
from .talker import Qwen3OmniMoeTalker
from .thinker import Qwen3OmniMoeThinker


def build_qwen3_omni_stage(model_stage, hf_config: dict, dtype, device, **kw):
    if kw.get("tiny") or (hf_config or {}).get("tiny"):
        cfg = Qwen3OmniConfig.tiny()
    elif hf_config:
        cfg = Qwen3OmniConfig.from_hf(hf_config)
    else:
        cfg = Qwen3OmniConfig()
    for k in ("num_hidden_layers",):          # benchmark / test override of the depth
        if kw.get("thinker_layers"):
            cfg.thinker.num_hidden_layers = int(kw["thinker_layers"])
            cfg.accept_hidden_layer = min(cfg.accept_hidden_layer, cfg.thinker.num_hidden_layers)
        if kw.get("talker_layers"):
            cfg.talker.num_hidden_layers = int(kw["talker_layers"])
    stage = (model_stage or "thinker").lower()
    if stage == "thinker":
        return Qwen3OmniMoeThinker(cfg, dtype, device)
    if stage == "talker":
        return Qwen3OmniMoeTalker(cfg, dtype, device)
    if stage == "code2wav":
        return Qwen3OmniCode2Wav(cfg, dtype, device)
    raise ValueError(f"unknown model_stage {model_stage!r} for Qwen3-Omni")
