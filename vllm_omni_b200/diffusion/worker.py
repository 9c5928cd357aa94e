"""One diffusion worker per GPU.

``DiffusionWorker`` binds a device, joins the process groups, loads the pipeline and runs
requests; ``WorkerProc`` is the process body used by the multi-process executor: it serves
RPCs from a broadcast queue, rank 0 returns results
(vllm_omni/diffusion/worker/diffusion_worker.py:48-485).  A heartbeat counter published
to the executor lets the engine detect a dead or stalled worker without touching the GPU.
"""
from __future__ import annotations

import importlib
import os
import threading
import time
import traceback
from typing import Any

import torch

from ..logger import init_logger
from .data import DiffusionOutput, OmniDiffusionConfig
from .model_runner import DiffusionModelRunner
from .request import OmniDiffusionRequest

logger = init_logger(__name__)


class DiffusionWorker:
    def __init__(self, local_rank: int, rank: int, od_config: OmniDiffusionConfig):
        self.local_rank, self.rank, self.od_config = local_rank, rank, od_config
        self.device = None
        self.model_runner: DiffusionModelRunner | None = None
        self.lora_manager = None
        self._sleeping_level = 0
        self._offloaded: dict[str, torch.Tensor] = {}
        self.profiler = None

    # ------------------------------------------------------------------ set-up
    def init_device(self, external_launcher: bool = False):
        cfg = self.od_config
        use_cuda = torch.cuda.is_available() and cfg.device != "cpu"
        self.device = torch.device("cuda", self.local_rank) if use_cuda else torch.device("cpu")
        if use_cuda:
            torch.cuda.set_device(self.device)
        world = cfg.parallel_config.world_size
        if world > 1 or external_launcher:
            from ..parallel import parallel_state as ps
            if not external_launcher:
                os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
                os.environ["MASTER_PORT"] = str(cfg.master_port)
                os.environ["RANK"], os.environ["LOCAL_RANK"] = str(self.rank), str(self.local_rank)
                os.environ["WORLD_SIZE"] = str(world)
            ps.init_distributed_environment(world_size=world, rank=self.rank, local_rank=self.local_rank,
                                            backend="nccl" if use_cuda else "gloo", timeout_s=cfg.dist_timeout)
            pc = cfg.parallel_config
            if not ps.model_parallel_is_initialized():
                ps.initialize_model_parallel(
                    data_parallel_size=pc.data_parallel_size, cfg_parallel_size=pc.cfg_parallel_size,
                    sequence_parallel_size=pc.sequence_parallel_size, ulysses_degree=pc.ulysses_degree,
                    ring_degree=pc.ring_degree, tensor_parallel_size=pc.tensor_parallel_size,
                    pipeline_parallel_size=pc.pipeline_parallel_size,
                    vae_patch_parallel_size=pc.vae_patch_parallel_size, backend="nccl" if use_cuda else "gloo")
        self.model_runner = DiffusionModelRunner(cfg, self.device)

    def load_model(self):
        self.model_runner.load_model()
        if self.od_config.lora_path:
            from .lora.manager import DiffusionLoRAManager
            self.lora_manager = DiffusionLoRAManager(self.model_runner.pipeline, max_cached=self.od_config.max_cpu_loras)
            self.lora_manager.add_adapter_from_path("default", self.od_config.lora_path, self.od_config.lora_scale)
            self.lora_manager.set_active(["default"])

    # ------------------------------------------------------------------ serving
    def generate(self, req: OmniDiffusionRequest) -> DiffusionOutput:
        return self.execute_model(req)

    def execute_model(self, req: OmniDiffusionRequest) -> DiffusionOutput:
        if self._sleeping_level:
            return DiffusionOutput(error="worker is asleep; call wake_up() first")
        lr = req.sampling_params.lora_request
        if lr is not None:
            self._ensure_lora().activate_request(lr, req.sampling_params.lora_scale)
        return self.model_runner.execute_model(req)

    # ------------------------------------------------------------------ LoRA
    def _ensure_lora(self):
        if self.lora_manager is None:
            from .lora.manager import DiffusionLoRAManager
            self.lora_manager = DiffusionLoRAManager(self.model_runner.pipeline, max_cached=self.od_config.max_cpu_loras)
        return self.lora_manager

    def add_lora(self, lora_request, scale: float = 1.0) -> bool:
        return self._ensure_lora().add_adapter_from_request(lora_request, scale)

    def remove_lora(self, lora_id: int) -> bool:
        return self._ensure_lora().remove_adapter(lora_id)

    def list_loras(self) -> list[int]:
        return self._ensure_lora().list_adapters()

    def pin_lora(self, lora_id: int) -> bool:
        return self._ensure_lora().pin_adapter(lora_id)

    # ------------------------------------------------------------------ sleep mode
    def sleep(self, level: int = 1) -> int:
        """Level 1 moves the weights to pinned host memory, level 2 discards them; both
        release the GPU memory.  Returns the number of bytes freed."""
        if self._sleeping_level or self.device.type != "cuda":
            self._sleeping_level = level
            return 0
        freed = 0
        for name, p in self.model_runner.pipeline.named_parameters():
            freed += p.numel() * p.element_size()
            if level == 1:
                host = torch.empty(p.shape, dtype=p.dtype, pin_memory=self.od_config.pin_cpu_memory)
                host.copy_(p.data, non_blocking=True)
                self._offloaded[name] = host
            p.data = torch.empty(0, dtype=p.dtype, device=self.device)
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        self._sleeping_level = level
        return freed

    def wake_up(self, tags: list[str] | None = None) -> bool:
        if not self._sleeping_level:
            return True
        if self._sleeping_level == 2 and not self._offloaded and self.device.type == "cuda":
            self.model_runner.load_model()        # weights were discarded: reload
        else:
            params = dict(self.model_runner.pipeline.named_parameters())
            for name, host in self._offloaded.items():
                params[name].data = host.to(self.device, non_blocking=True)
            if self.device.type == "cuda":
                torch.cuda.synchronize()
        self._offloaded.clear()
        self._sleeping_level = 0
        return True

    def load_weights(self, weights) -> set:
        return self.model_runner.pipeline.load_weights(weights)

    # ------------------------------------------------------------------ profiling
    def start_profile(self, trace_dir: str | None = None) -> bool:
        from .profiler import TorchProfiler
        self.profiler = TorchProfiler(trace_dir, rank=self.rank)
        self.profiler.start()
        return True

    def stop_profile(self):
        if self.profiler is None:
            return None
        path = self.profiler.stop()
        self.profiler = None
        return path

    def check_health(self) -> bool:
        return True

    def shutdown(self):
        try:
            from ..parallel import parallel_state as ps
            if torch.distributed.is_initialized():
                ps.destroy_distributed_environment()
        except Exception:
            pass


class WorkerWrapperBase:
    """Resolves ``worker_extension_cls`` (a dotted path) and mixes it into the worker so that
    custom pipelines can add RPC methods (vllm_omni/diffusion/worker/diffusion_worker.py:488-683)."""

    def __init__(self, local_rank: int, rank: int, od_config: OmniDiffusionConfig):
        cls = DiffusionWorker
        ext = od_config.worker_extension_cls
        if ext:
            mod, _, name = ext.rpartition(".")
            ext_cls = getattr(importlib.import_module(mod), name)
            cls = type(f"{name}Worker", (ext_cls, DiffusionWorker), {})
        self.worker = cls(local_rank, rank, od_config)

    def __getattr__(self, item):
        return getattr(self.worker, item)


class CustomPipelineWorkerExtension:
    """Mix-in giving workers ``re_init_pipeline`` for ``load_format='custom_pipeline'``."""

    def re_init_pipeline(self, pipeline_cls_path: str, **kwargs):
        mod, _, name = pipeline_cls_path.rpartition(".")
        cls = getattr(importlib.import_module(mod), name)
        self.model_runner.pipeline = cls(self.od_config, device=self.device, **kwargs)
        return True


def worker_main(local_rank: int, rank: int, od_config: OmniDiffusionConfig, cmd_q, res_q, ready_conn, heartbeat):
    """Process body: handshake, then serve RPCs until a shutdown message."""
    os.environ["OMNI_LOGGING_PREFIX"] = f"[diffusion-rank{rank}] "
    try:
        w = WorkerWrapperBase(local_rank, rank, od_config)
        w.init_device()
        w.load_model()
        ready_conn.send({"status": "ready", "rank": rank})
    except Exception as e:
        ready_conn.send({"status": "error", "rank": rank, "error": f"{e}\n{traceback.format_exc()}"})
        return
    finally:
        ready_conn.close()
    # liveness: a side thread bumps the shared counter a few times per second whatever the main
    # thread is doing, so the engine can tell a long-running generation (counter moves) from a
    # frozen process (counter stands still)
    stop_beat = threading.Event()

    def _beat():
        while not stop_beat.wait(0.2):
            with heartbeat.get_lock():
                heartbeat.value += 1

    threading.Thread(target=_beat, name="omni-worker-heartbeat", daemon=True).start()
    while True:
        try:
            msg = cmd_q.get(timeout=0.5)
        except Exception:
            continue
        if msg.get("type") == "shutdown":
            break
        method, args, kwargs = msg["method"], msg.get("args", ()), msg.get("kwargs", {})
        try:
            out: Any = getattr(w, method)(*args, **kwargs)
            if isinstance(out, DiffusionOutput) and isinstance(out.output, torch.Tensor):
                out.output = out.output.detach().cpu()
            err = None
        except Exception as e:
            out, err = None, f"{type(e).__name__}: {e}\n{traceback.format_exc()}"
        if rank == msg.get("output_rank", 0) or msg.get("reply_all"):
            res_q.put({"id": msg["id"], "rank": rank, "result": out, "error": err})
    stop_beat.set()
    w.shutdown()
