"""Diffusion engine: request pre-processing, batching, execution, post-processing.

``step`` keeps the contract of the reference engine (vllm_omni/diffusion/diffusion_engine.py:
69-180: pre_process -> executor -> post_process -> ``OmniRequestOutput`` per prompt) and adds
what it lacks: requests of equal shape are batched into one denoising loop
(``max_batch_size``), ``abort`` works for queued requests, and a dead worker turns into a
typed error instead of a hang.
"""
from __future__ import annotations

import threading
import time
from collections import deque

import torch

from ..inputs.data import OmniDiffusionSamplingParams
from ..logger import init_logger
from ..outputs import OmniRequestOutput
from .data import OmniDiffusionConfig
from .executor import DiffusionExecutor
from .registry import get_post_process_func, get_pre_process_func, supports_audio_output, supports_video_output
from .request import OmniDiffusionRequest

logger = init_logger(__name__)


class DiffusionEngine:
    def __init__(self, od_config: OmniDiffusionConfig, warmup: bool = False):
        self.od_config = od_config
        self.pre_process_func = get_pre_process_func(od_config)
        self.post_process_func = get_post_process_func(od_config)
        self.executor = DiffusionExecutor.get_class(od_config)(od_config)
        self._aborted: set[str] = set()
        self._lock = threading.Lock()
        self._queue: deque = deque()
        if warmup:
            self._dummy_run()

    @classmethod
    def make_engine(cls, od_config: OmniDiffusionConfig, **kw) -> "DiffusionEngine":
        return cls(od_config, **kw)

    # ------------------------------------------------------------------ serving
    def step(self, request: OmniDiffusionRequest) -> list[OmniRequestOutput]:
        live = [i for i, rid in enumerate(request.request_ids or [""] * len(request.prompts))
                if rid not in self._aborted]
        if request.request_ids and len(live) < len(request.prompts):
            request = OmniDiffusionRequest([request.prompts[i] for i in live], request.sampling_params,
                                           [request.request_ids[i] for i in live])
            if not request.prompts:
                return []
        pre_ms = 0.0
        if self.pre_process_func is not None:
            t = time.perf_counter()
            request = self.pre_process_func(request)
            pre_ms = (time.perf_counter() - t) * 1e3
        t_exec = time.perf_counter()
        output = self.executor.add_req(request)
        exec_ms = (time.perf_counter() - t_exec) * 1e3
        if output is None:            # non-output rank of an SPMD launch
            return []
        if output.error:
            raise RuntimeError(output.error)
        sp = request.sampling_params
        n_out = sp.num_outputs_per_prompt
        ids = request.request_ids or [""] * len(request.prompts)
        if output.output is None:
            return [OmniRequestOutput.from_diffusion(ids[i], [], p, {}) for i, p in enumerate(request.prompts)]
        t = time.perf_counter()
        outs = self.post_process_func(output.output) if self.post_process_func else output.output
        post_ms = (time.perf_counter() - t) * 1e3
        if not isinstance(outs, list):
            outs = [outs]
        metrics = {"image_num": int(n_out), "resolution": int(sp.resolution), "postprocess_time_ms": post_ms,
                   "preprocessing_time_ms": pre_ms, "execute_time_ms": exec_ms, **(output.metrics or {})}
        name = self.od_config.model_class_name
        results = []
        for i, prompt in enumerate(request.prompts):
            chunk = outs[i * n_out:(i + 1) * n_out]
            if supports_audio_output(name):
                mm = {"audio": chunk[0] if len(chunk) == 1 else chunk}
                if "sample_rate" in metrics:
                    mm["sample_rate"] = int(metrics["sample_rate"])
                results.append(OmniRequestOutput.from_diffusion(ids[i], [], prompt, metrics, output.trajectory_latents, mm,
                                                                "audio"))
            elif supports_video_output(name):
                results.append(OmniRequestOutput.from_diffusion(ids[i], [], prompt, metrics, output.trajectory_latents,
                                                                {"video": chunk[0] if len(chunk) == 1 else chunk},
                                                                "video"))
            else:
                results.append(OmniRequestOutput.from_diffusion(ids[i], chunk, prompt, metrics,
                                                                output.trajectory_latents))
        return results

    def step_batch(self, requests: list[OmniDiffusionRequest]) -> list[list[OmniRequestOutput]]:
        """Run several single-prompt requests; those whose sampling parameters agree (size,
        steps, guidance) share one denoising loop of up to ``max_batch_size`` prompts."""
        def key(r):
            s = r.sampling_params
            return (s.height, s.width, s.num_inference_steps, s.true_cfg_scale, s.guidance_scale, s.num_frames,
                    s.num_outputs_per_prompt, s.seed is None)
        groups: dict = {}
        for idx, r in enumerate(requests):
            groups.setdefault(key(r), []).append(idx)
        results: list = [None] * len(requests)
        mb = max(1, self.od_config.max_batch_size)
        for idxs in groups.values():
            for c in range(0, len(idxs), mb):
                chunk = idxs[c:c + mb]
                if len(chunk) == 1 or requests[chunk[0]].sampling_params.seed is not None:
                    for i in chunk:
                        results[i] = self.step(requests[i])
                    continue
                merged = OmniDiffusionRequest([p for i in chunk for p in requests[i].prompts],
                                              requests[chunk[0]].sampling_params,
                                              [rid for i in chunk for rid in (requests[i].request_ids or [""])])
                outs = self.step(merged)
                pos = 0
                for i in chunk:
                    n = len(requests[i].prompts)
                    results[i] = outs[pos:pos + n]
                    pos += n
        return results

    def abort(self, request_ids) -> None:
        """Queued requests with these ids are dropped before they reach a worker; a request
        that is already inside its denoising loop runs to completion."""
        if isinstance(request_ids, str):
            request_ids = [request_ids]
        with self._lock:
            self._aborted.update(request_ids)

    def clear_aborted(self, request_id: str) -> None:
        with self._lock:
            self._aborted.discard(request_id)

    # ------------------------------------------------------------------ management
    def collective_rpc(self, method: str, timeout: float | None = None, args=(), kwargs=None,
                       unique_reply_rank: int | None = None):
        return self.executor.collective_rpc(method, args=args, kwargs=kwargs, timeout=timeout,
                                            unique_reply_rank=unique_reply_rank)

    def check_health(self) -> bool:
        return self.executor.check_health()

    def start_profile(self, trace_dir: str | None = None):
        return self.collective_rpc("start_profile", kwargs={"trace_dir": trace_dir})

    def stop_profile(self):
        return self.collective_rpc("stop_profile")

    def sleep(self, level: int = 1):
        return self.collective_rpc("sleep", kwargs={"level": level})

    def wake_up(self, tags=None):
        return self.collective_rpc("wake_up", kwargs={"tags": tags})

    def _dummy_run(self):
        """One-step warm-up at the default resolution (allocates workspaces, loads kernels)."""
        size = 1024 if self.od_config.device != "cpu" and torch.cuda.is_available() else 64
        sp = OmniDiffusionSamplingParams(height=size, width=size, num_inference_steps=1, seed=0,
                                         output_type="latent")
        self.step(OmniDiffusionRequest(["warmup"], sp, ["_warmup"]))

    def close(self):
        self.executor.shutdown()

    shutdown = close
