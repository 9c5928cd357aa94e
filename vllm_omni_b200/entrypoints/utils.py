"""Stage-config loading.

Schema (docs/configuration/stage_configs.md:34-133 of the reference): top-level
``async_chunk``, ``runtime{defaults, connectors, edges}`` and ``stage_args`` — a list of
stages with ``stage_id, stage_type (llm|diffusion), runtime{process, devices,
max_batch_size, requires_multimodal_data}, engine_args{...}, engine_input_source,
custom_process_input_func, final_output, final_output_type, is_comprehension,
default_sampling_params, input_connectors, output_connectors``.  A small typed loader
replaces OmegaConf (vllm_omni/entrypoints/utils.py:120-236).
"""
from __future__ import annotations

import copy
import importlib
import json
import os
from dataclasses import dataclass, field
from typing import Any, Callable

import yaml

PKG_STAGE_CONFIG_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "stage_configs")


@dataclass
class StageConfig:
    stage_id: int = 0
    stage_type: str = "llm"
    runtime: dict[str, Any] = field(default_factory=dict)
    engine_args: dict[str, Any] = field(default_factory=dict)
    engine_input_source: list[int] = field(default_factory=list)
    custom_process_input_func: str | None = None
    final_output: bool = False
    final_output_type: str | None = None
    is_comprehension: bool = False
    default_sampling_params: dict[str, Any] = field(default_factory=dict)
    input_connectors: dict[str, Any] | None = None
    output_connectors: dict[str, Any] | None = None

    @classmethod
    def from_dict(cls, d: dict) -> "StageConfig":
        known = {k: copy.deepcopy(v) for k, v in d.items() if k in cls.__dataclass_fields__}
        sc = cls(**known)
        sc.engine_input_source = [int(x) for x in (sc.engine_input_source or [])]
        sc.runtime = dict(sc.runtime or {})
        sc.engine_args = dict(sc.engine_args or {})
        if sc.stage_type not in ("llm", "diffusion"):
            raise ValueError(f"stage {sc.stage_id}: stage_type must be 'llm' or 'diffusion', got {sc.stage_type!r}")
        return sc


@dataclass
class OmniPipelineConfig:
    stages: list[StageConfig]
    async_chunk: bool = False
    runtime: dict[str, Any] = field(default_factory=dict)


def _deep_merge(base: dict, over: dict) -> dict:
    out = copy.deepcopy(base)
    for k, v in over.items():
        if isinstance(v, dict) and isinstance(out.get(k), dict):
            out[k] = _deep_merge(out[k], v)
        else:
            out[k] = copy.deepcopy(v)
    return out


def load_stage_configs_from_yaml(path: str, base_engine_args: dict | None = None) -> OmniPipelineConfig:
    with open(path) as f:
        raw = yaml.safe_load(f) or {}
    return load_stage_configs_from_dict(raw, base_engine_args)


def load_stage_configs_from_dict(raw: dict, base_engine_args: dict | None = None) -> OmniPipelineConfig:
    base_engine_args = {k: v for k, v in (base_engine_args or {}).items() if v is not None}
    stages = []
    async_chunk = bool(raw.get("async_chunk", False))
    for sd in raw.get("stage_args", []):
        sd = copy.deepcopy(sd)
        sd["engine_args"] = _deep_merge(base_engine_args, sd.get("engine_args") or {})
        rt = sd.setdefault("runtime", {})
        if "max_batch_size" in rt:
            sd["engine_args"].setdefault("max_num_seqs", rt["max_batch_size"])
        sd["engine_args"]["async_chunk"] = async_chunk
        stages.append(StageConfig.from_dict(sd))
    ids = [s.stage_id for s in stages]
    if ids != list(range(len(ids))):
        raise ValueError(f"stage_ids must be 0..N-1 in order, got {ids}")
    for s in stages:
        for src in s.engine_input_source:
            if src >= s.stage_id:
                raise ValueError(f"stage {s.stage_id} takes input from stage {src}; sources must precede it")
    return OmniPipelineConfig(stages, async_chunk, dict(raw.get("runtime") or {}))


def get_model_type(model: str | None) -> str | None:
    """``model_type`` of a local HF directory's config.json (None when absent)."""
    if not model or not os.path.isdir(model):
        return None
    p = os.path.join(model, "config.json")
    if not os.path.exists(p):
        return None
    with open(p) as f:
        return json.load(f).get("model_type")


_NAME_HINTS = (("qwen3-omni", "qwen3_omni_moe"), ("qwen3_omni", "qwen3_omni_moe"), ("qwen2.5-omni", "qwen2_5_omni"),
               ("qwen2_5_omni", "qwen2_5_omni"), ("qwen3-tts", "qwen3_tts"), ("qwen3_tts", "qwen3_tts"),
               ("bagel", "bagel"))


def resolve_model_config_path(model: str | None) -> str | None:
    """model -> packaged ``stage_configs/{model_type}.yaml`` (None for plain diffusion models)."""
    mt = get_model_type(model)
    if mt is None and model:
        low = model.lower()
        for hint, name in _NAME_HINTS:
            if hint in low:
                mt = name
                break
    if mt is None:
        return None
    p = os.path.join(PKG_STAGE_CONFIG_DIR, f"{mt}.yaml")
    return p if os.path.exists(p) else None


def resolve_callable(path: str | None) -> Callable | None:
    if not path:
        return None
    mod, _, name = path.rpartition(".")
    # stage configs written for the reference name its modules; map them onto this package
    mod = mod.replace("vllm_omni.model_executor.stage_input_processors", "vllm_omni_b200.models.stage_input_processors")
    return getattr(importlib.import_module(mod), name)


def inject_omni_kv_config(stage_cfgs: list[StageConfig]) -> None:
    """Tell a KV-sending stage and its consumers about each other
    (vllm_omni/entrypoints/utils.py:21)."""
    for sc in stage_cfgs:
        kv = sc.engine_args.get("omni_kv_config")
        if not kv:
            continue
        kv.setdefault("stage_id", sc.stage_id)
        if kv.get("need_send_cache"):
            kv.setdefault("to_stages", [s.stage_id for s in stage_cfgs if sc.stage_id in s.engine_input_source])
        if kv.get("need_recv_cache"):
            kv.setdefault("from_stage", sc.engine_input_source[0] if sc.engine_input_source else None)


def voices_of_checkpoint(model: str | None) -> list[str]:
    """Named voices of a speech checkpoint: the keys of ``talker_config.spk_id`` (Qwen3-TTS) or
    ``talker_config.speaker_id`` (Qwen3-Omni) in its ``config.json``; [] when there is none."""
    if not model or not os.path.isdir(model):
        return []
    try:
        with open(os.path.join(model, "config.json")) as f:
            tk = json.load(f).get("talker_config") or {}
    except (OSError, ValueError):
        return []
    table = tk.get("spk_id") or tk.get("speaker_id") or {}
    return list(table) if isinstance(table, dict) else []
