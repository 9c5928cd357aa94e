"""Configuration and result types of the diffusion engine.

Field names and validation rules follow the reference
(vllm_omni/diffusion/data.py:28-99 parallel config, :129-241 cache config, :245-528 engine
config, :532 output) so that YAML stage configs and CLI flags carry over.
"""
from __future__ import annotations

import os
import random
from dataclasses import dataclass, field, fields
from typing import Any, Callable

import torch


@dataclass
class DiffusionParallelConfig:
    pipeline_parallel_size: int = 1
    data_parallel_size: int = 1
    tensor_parallel_size: int = 1
    sequence_parallel_size: int | None = None
    ulysses_degree: int = 1
    ring_degree: int = 1
    cfg_parallel_size: int = 1
    vae_patch_parallel_size: int = 1

    def __post_init__(self):
        if self.sequence_parallel_size is None:
            self.sequence_parallel_size = self.ulysses_degree * self.ring_degree
        for n in ("pipeline_parallel_size", "data_parallel_size", "tensor_parallel_size", "sequence_parallel_size",
                  "ulysses_degree", "ring_degree", "cfg_parallel_size", "vae_patch_parallel_size"):
            if getattr(self, n) <= 0:
                raise ValueError(f"{n} must be > 0")
        if self.cfg_parallel_size not in (1, 2):
            raise ValueError(f"CFG parallel size must be 1 or 2, but got {self.cfg_parallel_size}")
        if self.sequence_parallel_size != self.ulysses_degree * self.ring_degree:
            raise ValueError("sequence_parallel_size must equal ulysses_degree * ring_degree, got "
                             f"{self.sequence_parallel_size} != {self.ulysses_degree} * {self.ring_degree}")
        self.world_size = (self.pipeline_parallel_size * self.data_parallel_size * self.tensor_parallel_size *
                           self.ulysses_degree * self.ring_degree * self.cfg_parallel_size)

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "DiffusionParallelConfig":
        if not isinstance(data, dict):
            raise TypeError(f"Expected parallel config dict, got {type(data)!r}")
        return cls(**data)


@dataclass
class TransformerConfig:
    """Raw ``transformer/config.json`` dictionary with attribute access."""
    params: dict[str, Any] = field(default_factory=dict)

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "TransformerConfig":
        if not isinstance(data, dict):
            raise TypeError(f"Expected transformer config dict, got {type(data)!r}")
        return cls(params=dict(data))

    def to_dict(self):
        return dict(self.params)

    def get(self, key, default=None):
        return self.params.get(key, default)

    def __getattr__(self, item):
        params = object.__getattribute__(self, "params")
        try:
            return params[item]
        except KeyError as exc:
            raise AttributeError(item) from exc


@dataclass
class DiffusionCacheConfig:
    # TeaCache
    rel_l1_thresh: float = 0.2
    coefficients: list[float] | None = None
    # DBCache / TaylorSeer / SCM (cache-dit vocabulary)
    Fn_compute_blocks: int = 1
    Bn_compute_blocks: int = 0
    max_warmup_steps: int = 4
    max_cached_steps: int = -1
    residual_diff_threshold: float = 0.24
    max_continuous_cached_steps: int = 3
    enable_taylorseer: bool = False
    taylorseer_order: int = 1
    scm_steps_mask_policy: str | None = None
    scm_steps_policy: str = "dynamic"
    num_inference_steps: int | None = None
    _extra_params: dict[str, Any] = field(default_factory=dict, repr=False)

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "DiffusionCacheConfig":
        if not isinstance(data, dict):
            raise TypeError(f"Expected cache config dict, got {type(data)!r}")
        names = {f.name for f in fields(cls)}
        known = {k: v for k, v in data.items() if k in names and not k.startswith("_")}
        extra = {k: v for k, v in data.items() if k not in names}
        return cls(**known, _extra_params=extra)

    def __getattr__(self, item):
        if item == "_extra_params" or item.startswith("_"):
            raise AttributeError(item)
        extra = object.__getattribute__(self, "_extra_params")
        if item in extra:
            return extra[item]
        raise AttributeError(item)


@dataclass
class OmniDiffusionConfig:
    model: str | None = None
    model_class_name: str | None = None
    dtype: torch.dtype = torch.bfloat16
    tf_model_config: TransformerConfig = field(default_factory=TransformerConfig)
    attention_backend: str | None = None          # accepted for compatibility; there is one backend
    cache_strategy: str = "none"
    parallel_config: DiffusionParallelConfig = field(default_factory=DiffusionParallelConfig)
    cache_backend: str = "none"                   # none | tea_cache | cache_dit
    cache_config: DiffusionCacheConfig | dict[str, Any] = field(default_factory=dict)
    enable_cache_dit_summary: bool = False
    distributed_executor_backend: str = "mp"
    nccl_port: int | None = None
    trust_remote_code: bool = False
    revision: str | None = None
    num_gpus: int | None = None
    dist_timeout: int | None = None
    lora_path: str | None = None
    lora_scale: float = 1.0
    max_cpu_loras: int | None = None
    output_type: str = "pil"
    enable_cpu_offload: bool = False
    enable_layerwise_offload: bool = False
    pin_cpu_memory: bool = True
    vae_use_slicing: bool = False
    vae_use_tiling: bool = False
    enforce_eager: bool = False                   # True disables CUDA-graph capture of the step
    enable_sleep_mode: bool = False
    master_port: int | None = None
    worker_extension_cls: str | None = None
    custom_pipeline_args: dict[str, Any] | None = None
    diffusion_load_format: str = "default"        # default | custom_pipeline | dummy
    host: str | None = None
    port: int | None = None
    model_paths: dict[str, str] = field(default_factory=dict)
    vae_config: dict[str, Any] = field(default_factory=dict)   # vae/config.json of the checkpoint (or overrides)
    override_transformer_cls_name: str | None = None
    boundary_ratio: float | None = None
    flow_shift: float | None = None
    supports_multimodal_inputs: bool = False
    log_level: str = "info"
    omni_kv_config: dict[str, Any] = field(default_factory=dict)
    quantization: str | None = None
    quantization_config: Any = None
    max_batch_size: int = 1                       # requests batched into one denoising loop
    device: str | None = None                     # "cpu" runs the PyTorch restatement (tests, config 1)
    seed: int = 0

    def __post_init__(self):
        if isinstance(self.parallel_config, dict):
            self.parallel_config = DiffusionParallelConfig.from_dict(self.parallel_config)
        if isinstance(self.tf_model_config, dict):
            self.tf_model_config = TransformerConfig.from_dict(self.tf_model_config)
        if isinstance(self.dtype, str):
            self.dtype = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float16": torch.float16,
                          "fp16": torch.float16, "float32": torch.float32, "fp32": torch.float32,
                          "auto": torch.bfloat16}[self.dtype]
        env_backend = os.environ.get("DIFFUSION_CACHE_BACKEND")
        if env_backend and self.cache_backend in (None, "none"):
            self.cache_backend = env_backend
        if self.cache_backend is None:
            self.cache_backend = "none"
        if isinstance(self.cache_config, dict):
            self.cache_config = DiffusionCacheConfig.from_dict(self.cache_config)
        if self.num_gpus is None:
            self.num_gpus = self.parallel_config.world_size
        if self.num_gpus < self.parallel_config.world_size:
            raise ValueError(f"num_gpus ({self.num_gpus}) < parallel world size ({self.parallel_config.world_size})")
        if self.master_port is None:
            self.master_port = 30005 + random.randint(0, 1000)
        if self.enable_cpu_offload and self.enable_layerwise_offload:
            raise ValueError("enable_cpu_offload and enable_layerwise_offload are mutually exclusive")

    @classmethod
    def from_kwargs(cls, **kwargs) -> "OmniDiffusionConfig":
        names = {f.name for f in fields(cls)}
        if "parallel_config" not in kwargs:
            pc = {k: kwargs.pop(k) for k in list(kwargs) if k in {f.name for f in fields(DiffusionParallelConfig)}}
            if pc:
                kwargs["parallel_config"] = DiffusionParallelConfig(**pc)
        return cls(**{k: v for k, v in kwargs.items() if k in names})


@dataclass
class DiffusionOutput:
    output: Any = None
    trajectory_timesteps: list | None = None
    trajectory_latents: torch.Tensor | None = None
    trajectory_decoded: list | None = None
    error: str | None = None
    post_process_func: Callable[..., Any] | None = None
    metrics: dict[str, Any] = field(default_factory=dict)
