"""``Omni`` — blocking offline entry point over one or more stages.

``Omni(model, **kwargs).generate(prompts, sampling_params_list)`` mirrors the reference
(vllm_omni/entrypoints/omni.py:100-914): a stage-config YAML (or, for a diffusers-style
model, a synthesised single diffusion stage, omni.py:171-207) defines the stages; requests
enter stage 0 and each stage's outputs are turned into the next stage's inputs by the stage's
input processor; results of stages marked ``final_output`` are returned.

Stages are logical here: each owns its GPUs and a scheduler, and lives either in this process
(single-stage pipelines and tests) or in a worker process (``runtime.process: true``).  Data
between stages moves through an OmniConnector.
"""
from __future__ import annotations

import time
import uuid
from typing import Any, Sequence

from ..inputs.data import OmniDiffusionSamplingParams, OmniPromptType
from ..logger import init_logger
from ..outputs import OmniRequestOutput

logger = init_logger(__name__)


class OmniBase:
    def __init__(self, model: str | None = None, stage_configs_path: str | None = None, log_stats: bool = False,
                 stage_init_timeout: int = 300, shm_threshold_bytes: int = 65536, worker_backend: str = "mp",
                 ray_address: str | None = None, batch_timeout: int = 10, init_timeout: int = 300,
                 log_file: str | None = None, **kwargs: Any):
        from .stage_runtime import build_stages
        self.model = model
        self.log_stats = log_stats
        self.log_file = log_file
        self.kwargs = kwargs
        self.stage_list, self.connectors, self.stage_configs = build_stages(
            model, stage_configs_path, kwargs, stage_init_timeout=stage_init_timeout,
            shm_threshold_bytes=shm_threshold_bytes, worker_backend=worker_backend, batch_timeout=batch_timeout)
        from ..metrics.stats import OrchestratorAggregator
        self.metrics = OrchestratorAggregator(len(self.stage_list), log_stats, log_file)
        if len(self.stage_list) > 1:
            # Stages that run as threads of this process share one interpreter lock.  A stage loop that comes
            # back from a device wait must not sit out another thread's whole 5 ms slice before its next launch.
            import sys
            sys.setswitchinterval(min(sys.getswitchinterval(), 0.0005))
        self._closed = False

    @property
    def num_stages(self) -> int:
        return len(self.stage_list)

    @property
    def mm_processor_kwargs(self) -> dict:
        """How chat-request images / audio are turned into thinker inputs for this model (server side)."""
        if getattr(self, "_mm_kwargs", None) is None:
            from ..inputs.omni_processor import processor_kwargs_for
            self._mm_kwargs = processor_kwargs_for(self.model, getattr(self.stage_configs, "stages", None))
        return self._mm_kwargs

    def start_profile(self, stages: Sequence[int] | None = None, trace_dir: str | None = None):
        for s in self.stage_list:
            if stages is None or s.stage_id in stages:
                s.start_profile(trace_dir)

    def stop_profile(self, stages: Sequence[int] | None = None):
        return [s.stop_profile() for s in self.stage_list if stages is None or s.stage_id in stages]

    def check_health(self) -> bool:
        return all(s.check_health() for s in self.stage_list)

    def restart_stage(self, stage_id: int, timeout: float | None = None) -> None:
        """Replace a stage whose worker died (or hangs) by a fresh one with the same configuration:
        the old worker is stopped or terminated, a new worker loads the model again and the stage
        object is swapped in place, so stage ids, edges and connectors stay valid.  Requests that were
        inside the old worker are lost; the caller fails them (see ``AsyncOmni``)."""
        from .stage_runtime import OmniStage
        old = self.stage_list[stage_id]
        try:
            old.stop_stage_worker(join_timeout=1.0)
        except Exception:   # noqa: BLE001
            logger.exception("stopping stage %s before its restart failed", stage_id)
        new = OmniStage(old.cfg, old.model, batch_timeout_s=old.batch_timeout_s, stage_init_timeout=old.stage_init_timeout,
                        worker_backend=old.worker_backend, placement_group=getattr(old, "_placement_group", None))
        new.init_stage_worker()
        if not new.wait_ready(timeout):
            new.stop_stage_worker()
            raise RuntimeError(f"stage {stage_id} did not come back within its start-up limit")
        self.stage_list[stage_id] = new
        logger.warning("stage %s restarted", stage_id)

    def close(self):
        if self._closed:
            return
        self._closed = True
        for s in self.stage_list:
            try:
                s.stop_stage_worker()
            except Exception:
                logger.exception("stage %s failed to stop", s.stage_id)
        for c in (self.connectors or {}).values():
            try:
                c.cleanup_all()
            except Exception:
                pass

    shutdown = close

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Omni(OmniBase):
    def generate(self, prompts: OmniPromptType | Sequence[OmniPromptType],
                 sampling_params_list: Any = None, request_ids: Sequence[str] | None = None,
                 use_tqdm: bool = False) -> list[OmniRequestOutput]:
        from .orchestrator import run_generation
        if isinstance(prompts, (str, dict)):
            prompts = [prompts]
        prompts = list(prompts)
        if sampling_params_list is None:
            sampling_params_list = [s.default_sampling_params() for s in self.stage_list]
        elif not isinstance(sampling_params_list, (list, tuple)):
            sampling_params_list = [sampling_params_list]
        if len(sampling_params_list) != self.num_stages:
            if len(sampling_params_list) == 1 and self.num_stages > 1:
                raise ValueError(f"sampling_params_list needs one entry per stage ({self.num_stages})")
            if len(sampling_params_list) < self.num_stages:
                raise ValueError(f"expected {self.num_stages} sampling params, got {len(sampling_params_list)}")
        ids = list(request_ids) if request_ids else [f"req-{uuid.uuid4().hex[:10]}" for _ in prompts]
        t0 = time.time()
        outs = run_generation(self, prompts, list(sampling_params_list), ids)
        if self.log_stats:
            self.metrics.build_and_log_summary(time.time() - t0)
        return outs
