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
    stream_interval: int = 1              # generated tokens between progress reports of a running request (0 = none)
    stream_mm_interval: int = 1           # progress reports carry the model's streamed tensors on every n-th token only
    stream_output_keys: Any = None        # overrides the model's list of tensors that ride on progress reports
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
        # tensor-parallel followers are started by rank 0 with these three (engine/tp_worker.py)
        tp_rank = int(kwargs.pop("_tp_rank", 0))
        tp_port = kwargs.pop("_tp_port", None)
        tp_dev = kwargs.pop("_tp_device_index", None)
        self._spawn_kwargs = dict(kwargs, stage_id=stage_id)
        self.args = a = OmniEngineArgs.from_kwargs(model=model, stage_id=stage_id, **kwargs)
        dtype = _DTYPES[a.dtype] if isinstance(a.dtype, str) else a.dtype
        use_cuda = torch.cuda.is_available() and a.device != "cpu"
        tp = int(a.tensor_parallel_size or 1)
        self.tp_size, self.tp_rank, self.tp_control, self._tp_procs = tp, tp_rank, None, []
        tp_group = None
        if tp > 1:
            tp_group = self._join_tp_group(model, tp, tp_rank, tp_port, tp_dev, use_cuda)
        elif a.enable_expert_parallel:
            logger.info("stage %d: enable_expert_parallel has no effect with tensor_parallel_size=1", stage_id)
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
        if tp_group is not None:
            dec = getattr(self.model, "decoder", None)
            if dec is None or not hasattr(dec, "enable_tensor_parallel"):
                raise NotImplementedError(f"stage model {type(self.model).__name__} ({a.model_stage}) has no "
                                          "tensor-parallel decoder; set tensor_parallel_size: 1 for this stage")
            if a.async_chunk and stage_id > 0:
                raise NotImplementedError("a tensor-parallel stage cannot take its input as a chunk stream yet")
            dec.enable_tensor_parallel(tp_group, mode=os.environ.get("OMNI_TP_MODE"),
                                       expert_parallel=bool(a.enable_expert_parallel))
        chunk_adapter = kv_mgr = None
        if tp_rank > 0:
            a.async_chunk, a.omni_kv_config = False, {}       # connectors live on rank 0 only
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
        self.engine.stream_interval = int(a.stream_interval)
        self.engine.stream_mm_interval = int(a.stream_mm_interval)
        if a.stream_output_keys is not None:
            self.model.stream_output_keys = tuple(a.stream_output_keys)
        elif a.async_chunk and hasattr(self.model, "chunk_stream_keys"):
            # a producer of a chunk stream (the thinker under ``async_chunk``): its rows ride on every 8th token's report
            self.model.stream_output_keys = tuple(self.model.chunk_stream_keys)
            if a.stream_mm_interval <= 1:
                self.engine.stream_mm_interval = 8
        if tp_group is not None and hasattr(self.engine.runner, "tp_group"):
            self.engine.runner.tp_group = tp_group
        self._profiler = None

    # ------------------------------------------------------------------ tensor parallel group
    def _join_tp_group(self, model, tp, tp_rank, tp_port, tp_dev, use_cuda):
        """Rank 0 starts ranks 1..tp-1 (one process per GPU of this stage) and all join one group."""
        import torch.distributed as dist
        from ..engine import tp_worker
        if use_cuda and torch.cuda.device_count() < tp:
            raise ValueError(f"tensor_parallel_size={tp} but this stage sees {torch.cuda.device_count()} GPU(s); "
                             "list them under runtime.devices")
        if tp_rank == 0:
            if dist.is_initialized():
                raise NotImplementedError("tensor_parallel_size > 1 needs a process of its own for the stage "
                                          "(runtime.process: true): this process already has a process group")
            tp_port = tp_worker.free_port()
            devs = list(range(tp)) if use_cuda else [0] * tp
            self._tp_procs, readies, self._tp_errq = tp_worker.spawn_followers(tp, tp_port, model, self._spawn_kwargs, devs)
            tp_dev = devs[0]
        group = tp_worker.init_tp_process(tp_rank, tp, tp_port, use_cuda, tp_dev if tp_dev is not None else 0)
        self.tp_control = tp_worker.TPControl(group)
        return group

    # engine passthrough -------------------------------------------------
    def add_request(self, request_id, prompt, sampling_params: SamplingParams | None = None):
        req = self.engine.add_request(request_id, prompt, sampling_params)
        if self.tp_control is not None and self.tp_rank == 0:
            self.tp_control.pending_add.append((request_id, prompt, sampling_params))
        return req

    def step(self):
        if self.tp_control is not None and self.tp_rank == 0:
            if not self.engine.has_unfinished_requests() and not self.tp_control.pending_add \
                    and not self.tp_control.pending_abort:
                return []                     # nothing to run: do not wake the followers
            self._check_followers()
            self.tp_control.leader_step_message()
        return self.engine.step()

    def _check_followers(self):
        for p in self._tp_procs:
            if not p.is_alive():
                why = ""
                try:
                    why = self._tp_errq.get_nowait()
                except Exception:   # noqa: BLE001
                    pass
                raise RuntimeError(f"tensor-parallel worker {p.name} died (exit code {p.exitcode}) {why}")

    def has_unfinished_requests(self):
        return self.engine.has_unfinished_requests()

    def update_request(self, request_id: str, payload: dict) -> bool:
        """Late input for a running request (see ``LLMEngine.update_request``)."""
        return self.engine.update_request(request_id, payload)

    def abort_request(self, request_ids):
        if isinstance(request_ids, str):
            request_ids = [request_ids]
        self.engine.abort_request(request_ids)
        if self.tp_control is not None and self.tp_rank == 0:
            self.tp_control.pending_abort.extend(request_ids)

    def generate(self, prompts, sampling_params=None):
        """Blocking convenience wrapper: run the given prompts to completion."""
        import time
        if isinstance(prompts, (str, dict)):
            prompts = [prompts]
        sps = sampling_params if isinstance(sampling_params, (list, tuple)) else [sampling_params] * len(prompts)
        ids = [f"gen-{i}-{time.monotonic_ns()}" for i in range(len(prompts))]
        for rid, p, sp in zip(ids, prompts, sps):
            self.add_request(rid, p, sp)
        final = {}
        while len(final) < len(ids):
            for o in self.step():
                if o.finished and o.request_id in ids:
                    final[o.request_id] = o
        return [final[i] for i in ids]

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
        if self.tp_control is not None and self.tp_rank == 0 and self._tp_procs:
            self.tp_control.leader_shutdown()
            for p in self._tp_procs:
                p.join(timeout=10)
                if p.is_alive():
                    p.terminate()
            self._tp_procs = []
