"""``OmniLLM``: an AR (or one-shot generation) stage engine built from stage-config
``engine_args`` (vllm_omni/entrypoints/omni_llm.py, vllm_omni/engine/arg_utils.py):
``model_arch`` + ``model_stage`` pick the stage model, ``hf_config_name`` the sub-config,
``worker_type`` (ar | generation) the scheduler/runner pair, ``engine_output_type`` what the
stage hands downstream.  Tensor/expert parallel sizes map onto this framework's groups."""
from __future__ import annotations

import json
import os
import threading
from dataclasses import dataclass, field
from typing import Any

import torch

from ..engine.llm_engine import LLMEngine
from ..engine.tokenizer import get_tokenizer
from ..inputs.data import SamplingParams
from ..logger import init_logger
from ..models.registry import build_stage_model

logger = init_logger(__name__)
_BUILD_LOCK = threading.Lock()


@dataclass
class OmniEngineArgs:
    model: str | None = None
    stage_id: int = 0
    model_stage: str | None = None
    model_arch: str | None = None
    engine_output_type: str | None = None
    hf_config_name: str | None = None
    custom_process_next_stage_input_func: str | None = None
    stage_connector_spec: dict | None = None
    async_chunk: bool = False
    omni_kv_config: dict = field(default_factory=dict)
    worker_type: str = "ar"
    scheduler_cls: str | None = None
    dtype: Any = "bfloat16"
    device: str | None = None
    seed: int = 0
    gpu_memory_utilization: float = 0.9
    enforce_eager: bool = False
    trust_remote_code: bool = False
    enable_prefix_caching: bool = False
    max_num_batched_tokens: int = 8192
    max_num_seqs: int = 64
    max_model_len: int = 32768
    block_size: int = 16
    num_gpu_blocks: int | None = None
    tensor_parallel_size: int = 1
    enable_expert_parallel: bool = False
    distributed_executor_backend: str | None = None
    load_format: str = "auto"
    async_scheduling: bool = False
    model_overrides: dict = field(default_factory=dict)     # e.g. {"tiny": True} for tests

    @classmethod
    def from_kwargs(cls, **kw) -> "OmniEngineArgs":
        names = set(cls.__dataclass_fields__)
        extra = {k: v for k, v in kw.items() if k not in names}
        a = cls(**{k: v for k, v in kw.items() if k in names})
        if extra:
            logger.debug("ignored engine args: %s", sorted(extra))
        return a


_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32,
           "fp32": torch.float32, "auto": torch.bfloat16}


class OmniLLM:
    def __init__(self, model: str | None = None, stage_id: int = 0, **kwargs):
        self.args = a = OmniEngineArgs.from_kwargs(model=model, stage_id=stage_id, **kwargs)
        dtype = _DTYPES[a.dtype] if isinstance(a.dtype, str) else a.dtype
        use_cuda = torch.cuda.is_available() and a.device != "cpu"
        device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")
        if not use_cuda and dtype == torch.bfloat16:
            dtype = torch.float32
        hf_cfg = {}
        if model and os.path.isdir(model) and os.path.exists(os.path.join(model, "config.json")):
            with open(os.path.join(model, "config.json")) as f:
                hf_cfg = json.load(f)
            hf_cfg.setdefault("_model_dir", model)          # for models that keep sub-configs in sub-folders
        arch = a.model_arch or (hf_cfg.get("architectures") or ["Qwen3ForCausalLM"])[0]
        # stages that share a process are built on a thread pool and share torch's global generator:
        # seeding and random initialisation must not interleave, or the weights depend on thread timing
        with _BUILD_LOCK:
            torch.manual_seed(a.seed + 1000 * stage_id)
            self.model = build_stage_model(arch, a.model_stage, hf_cfg, dtype, device, **a.model_overrides)
        if model and os.path.isdir(model) and a.load_format not in ("dummy",):
            from ..diffusion.loader import _shard_files, safetensors_weights_iterator
            files = _shard_files(model)
            if files and hasattr(self.model, "load_weights"):
                n = len(self.model.load_weights(safetensors_weights_iterator(files)))
                if hasattr(self.model, "load_auxiliary"):          # weights kept beside the main checkpoint
                    n += self.model.load_auxiliary(model)
                logger.info("stage %d (%s): loaded %d tensors", stage_id, a.model_stage, n)
        self.model.eval()
        chunk_adapter = kv_mgr = None
        if a.async_chunk and a.stage_connector_spec:
            from ..connectors.chunk_transfer_adapter import OmniChunkTransferAdapter
            chunk_adapter = OmniChunkTransferAdapter.from_spec(a.stage_connector_spec, stage_id, a.model_stage)
        if a.omni_kv_config:
            from ..connectors.kv_transfer_manager import OmniKVTransferManager
            kv_mgr = OmniKVTransferManager.from_config(a.omni_kv_config)
        crit = (a.omni_kv_config or {}).get("kv_transfer_criteria")
        self.engine = LLMEngine(self.model, get_tokenizer(model, a.trust_remote_code), device, dtype,
                                block_size=a.block_size, num_gpu_blocks=a.num_gpu_blocks,
                                gpu_memory_utilization=a.gpu_memory_utilization, max_num_seqs=a.max_num_seqs,
                                max_num_batched_tokens=a.max_num_batched_tokens, max_model_len=a.max_model_len,
                                kv_transfer_criteria=crit, chunk_adapter=chunk_adapter, kv_transfer_manager=kv_mgr,
                                stage_id=stage_id, engine_output_type=a.engine_output_type)
        self._profiler = None

    # engine passthrough -------------------------------------------------
    def add_request(self, request_id, prompt, sampling_params: SamplingParams | None = None):
        return self.engine.add_request(request_id, prompt, sampling_params)

    def step(self):
        return self.engine.step()

    def has_unfinished_requests(self):
        return self.engine.has_unfinished_requests()

    def abort_request(self, request_ids):
        self.engine.abort_request(request_ids)

    def generate(self, prompts, sampling_params=None):
        return self.engine.generate(prompts, sampling_params)

    def start_profile(self, trace_dir=None):
        from ..diffusion.profiler import TorchProfiler
        self._profiler = TorchProfiler(trace_dir, rank=self.args.stage_id, template=f"stage{self.args.stage_id}")
        self._profiler.start()

    def stop_profile(self):
        if self._profiler is None:
            return None
        p, self._profiler = self._profiler.stop(), None
        return p

    def shutdown(self):
        pass
