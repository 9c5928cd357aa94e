"""Stage runtime: one ``OmniStage`` per YAML stage, its worker loop and engine adapters.

A stage owns an engine (AR ``LLMEngine`` or ``DiffusionEngine``), a task queue and a result
queue (vllm_omni/entrypoints/omni_stage.py:248-1375).  The same worker loop runs either on a
thread of the orchestrator process (``runtime.process: false`` — single-stage pipelines,
tests, SPMD launches) or in a spawned process (``runtime.process: true``).  Engines are
driven through a small adapter interface so that the loop does continuous batching for AR
stages (requests join and leave between engine steps) and window batching for diffusion
stages (requests with equal sampling parameters share one denoising loop).
"""
from __future__ import annotations

import multiprocessing as mp
import os
import queue
import threading
import time
import traceback
from dataclasses import asdict
from typing import Any

from ..inputs.data import OmniDiffusionSamplingParams, OmniTokensPrompt, SamplingParams
from ..logger import init_logger
from ..outputs import OmniRequestOutput
from .stage_utils import OmniStageTaskType, set_stage_devices, to_host
from .utils import (OmniPipelineConfig, StageConfig, inject_omni_kv_config, load_stage_configs_from_yaml,
                    resolve_callable, resolve_model_config_path)

logger = init_logger(__name__)


# ====================================================================== engine adapters
class StageEngineAdapter:
    def add_task(self, task: dict) -> None: ...
    def has_work(self) -> bool: ...
    def step(self) -> list[dict]: ...
    def abort(self, request_ids: list[str]) -> None: ...
    def update(self, task: dict) -> None: ...          # late input for a running request; ignored by default
    def shutdown(self) -> None: ...
    def start_profile(self, trace_dir=None): ...
    def stop_profile(self): ...


class DiffusionStageAdapter(StageEngineAdapter):
    def __init__(self, stage_id: int, model: str, engine_args: dict, max_batch_size: int, batch_timeout_s: float):
        from .omni_diffusion import OmniDiffusion
        args = {k: v for k, v in engine_args.items() if k not in ("model_stage", "async_chunk", "max_num_seqs")}
        args.setdefault("max_batch_size", max_batch_size)
        self.stage_id = stage_id
        self.engine = OmniDiffusion(model=args.pop("model", model), **args)
        self.max_batch_size = max(1, max_batch_size)
        self.batch_timeout_s = batch_timeout_s
        self.pending: list[dict] = []
        self._first_ts = 0.0
        self._batch_id = 0

    def add_task(self, task):
        if not self.pending:
            self._first_ts = time.monotonic()
        self.pending.append(task)

    def has_work(self):
        return bool(self.pending)

    def abort(self, request_ids):
        s = set(request_ids)
        self.pending = [t for t in self.pending if t["request_id"] not in s]
        self.engine.abort(request_ids)

    def step(self):
        if not self.pending:
            return []
        # wait (briefly) for the batch window to fill, like the reference's sync worker
        if len(self.pending) < self.max_batch_size and time.monotonic() - self._first_ts < self.batch_timeout_s \
                and self.max_batch_size > 1:
            return []
        from ..diffusion.request import OmniDiffusionRequest
        batch, self.pending = self.pending[:self.max_batch_size], self.pending[self.max_batch_size:]
        if self.pending:
            self._first_ts = time.monotonic()
        self._batch_id += 1
        results = []
        reqs = []
        for t in batch:
            sp = t.get("sampling_params") or OmniDiffusionSamplingParams()
            if isinstance(sp, dict):
                sp = OmniDiffusionSamplingParams(**sp)
            prompts = t["engine_inputs"]
            prompts = prompts if isinstance(prompts, list) else [prompts]
            reqs.append(OmniDiffusionRequest(prompts, sp, [t["request_id"]] * len(prompts)))
        t0 = time.perf_counter()
        try:
            outs = self.engine.engine.step_batch(reqs)
            err = None
        except Exception as e:
            outs, err = None, (f"{type(e).__name__}: {e}", traceback.format_exc())
        dt_ms = (time.perf_counter() - t0) * 1e3
        for i, t in enumerate(batch):
            if err is not None:
                results.append({"request_id": t["request_id"], "stage_id": self.stage_id, "error": err[0],
                                "error_tb": err[1]})
                continue
            results.append({"request_id": t["request_id"], "stage_id": self.stage_id, "engine_outputs": outs[i],
                            "finished": True,
                            "metrics": {"batch_id": self._batch_id, "batch_size": len(batch), "num_tokens_in": 0,
                                        "num_tokens_out": 0, "stage_gen_time_ms": dt_ms / len(batch),
                                        "diffusion_metrics": outs[i][0].metrics if outs[i] else {}}})
        return results

    def shutdown(self):
        self.engine.close()

    def start_profile(self, trace_dir=None):
        return self.engine.start_profile(trace_dir)

    def stop_profile(self):
        return self.engine.stop_profile()


class LLMStageAdapter(StageEngineAdapter):
    def __init__(self, stage_id: int, model: str, engine_args: dict, stream: bool = True):
        from .omni_llm import OmniLLM
        self.stage_id = stage_id
        self.llm = OmniLLM(model=engine_args.pop("model", model), stage_id=stage_id, **engine_args)
        self.stream = stream
        self._t0: dict[str, float] = {}

    def add_task(self, task):
        sp = task.get("sampling_params") or SamplingParams()
        if isinstance(sp, dict):
            sp = SamplingParams(**sp)
        inputs = task["engine_inputs"]
        inputs = inputs[0] if isinstance(inputs, list) and len(inputs) == 1 else inputs
        rid = task["request_id"]
        if task.get("chunk_index") is not None:      # several chunk sub-requests share one request id
            rid = f"{rid}#c{task['chunk_index']}"
        self._t0[rid] = time.perf_counter()
        self.llm.add_request(rid, inputs, sp)

    def has_work(self):
        return self.llm.has_unfinished_requests()

    def update(self, task):
        self.llm.update_request(task["request_id"], task.get("payload") or {})

    def abort(self, request_ids):
        ids = set(request_ids)
        full = [k for k in self._t0 if k.split("#c")[0] in ids] + list(request_ids)
        self.llm.abort_request(full)
        for r in full:
            self._t0.pop(r, None)

    def step(self):
        results = []
        try:
            outs = self.llm.step()
        except Exception as e:
            tb = traceback.format_exc()
            rids = list(self._t0)
            self.llm.abort_request(rids)
            self._t0.clear()
            return [{"request_id": r, "stage_id": self.stage_id, "error": f"{type(e).__name__}: {e}", "error_tb": tb}
                    for r in rids]
        for ro in outs:
            if not ro.finished and not self.stream:
                continue
            base_id = ro.request_id.split("#c")[0]
            full_id = ro.request_id
            ro.request_id = base_id
            res = {"request_id": base_id, "stage_id": self.stage_id, "engine_outputs": [ro],
                   "finished": ro.finished}
            if ro.finished:
                dt = (time.perf_counter() - self._t0.pop(full_id, time.perf_counter())) * 1e3
                res["metrics"] = {"batch_id": 0, "batch_size": 1, "num_tokens_in": len(ro.prompt_token_ids or []),
                                  "num_tokens_out": sum(len(o.token_ids) for o in ro.outputs),
                                  "stage_gen_time_ms": dt}
            results.append(res)
        return results

    def shutdown(self):
        self.llm.shutdown()

    def start_profile(self, trace_dir=None):
        return self.llm.start_profile(trace_dir)

    def stop_profile(self):
        return self.llm.stop_profile()


def make_adapter(cfg: StageConfig, model: str, batch_timeout_s: float) -> StageEngineAdapter:
    rt = cfg.runtime
    if cfg.stage_type == "diffusion":
        return DiffusionStageAdapter(cfg.stage_id, model, dict(cfg.engine_args), int(rt.get("max_batch_size", 1)),
                                     batch_timeout_s)
    args = dict(cfg.engine_args)
    if "stream_interval" not in args:
        # Progress reports cross a process boundary one message (and one device-to-host copy per tensor) each:
        # only the stage the client watches reports every step; a talker that feeds a chunked vocoder reports
        # once per chunk of frames; other intermediate stages report the finished request only.
        if cfg.final_output:
            args["stream_interval"] = 1
        elif args.get("async_chunk") and args.get("model_stage") == "talker":
            from ..models.stage_input_processors.qwen3_omni import CHUNK_FRAMES
            args["stream_interval"] = CHUNK_FRAMES
        else:
            args["stream_interval"] = 0
    return LLMStageAdapter(cfg.stage_id, model, args)


# adapters of stages that run on a thread of this process, by stage id (introspection, tests)
_INPROC_ADAPTERS: dict[int, StageEngineAdapter] = {}


def inproc_adapter(stage_id: int) -> StageEngineAdapter:
    return _INPROC_ADAPTERS[stage_id]


def _resolve_payload(task: dict, cache: dict) -> None:
    """Pull ``task['engine_inputs']`` through the edge connector when the orchestrator sent only a
    descriptor (process-separated stages).  Raises on a missing or corrupted payload; the worker turns
    that into an error result for this request."""
    cm = task.get("connector_meta")
    if cm is None or "engine_inputs" in task:
        return
    from ..connectors.adapter import try_recv_via_connector
    from ..connectors.factory import OmniConnectorFactory
    edge = (cm["from_stage"], cm["to_stage"])
    if edge not in cache:
        spec = cm.get("spec") or {"name": "SharedMemoryConnector"}
        if spec.get("name") == "FaultInjectionConnector":
            # faults are injected where the payload is produced; this end only has to read it
            spec = (spec.get("extra") or {}).get("inner") or {"name": "SharedMemoryConnector"}
            spec = {"name": spec} if isinstance(spec, str) else spec
        cache[edge] = OmniConnectorFactory.create(spec)
    try_recv_via_connector(cache[edge], task)


# ========================================================================= worker loop
def _stage_worker(cfg: StageConfig, model: str, in_q, out_q, batch_timeout_s: float, in_process: bool):
    """Body of a stage (thread or process)."""
    sid = cfg.stage_id
    if not in_process:
        os.environ["OMNI_LOGGING_PREFIX"] = f"[stage{sid}] "
        set_stage_devices(sid, cfg.runtime.get("devices"), in_process=False)
    try:
        adapter = make_adapter(cfg, model, batch_timeout_s)
    except Exception as e:
        out_q.put({"type": "stage_error", "stage_id": sid, "error": f"{type(e).__name__}: {e}",
                   "error_tb": traceback.format_exc()})
        return
    if in_process:
        _INPROC_ADAPTERS[sid] = adapter
    out_q.put({"type": "stage_ready", "stage_id": sid})
    paused = False
    held: list[dict] = []
    edge_connectors: dict = {}          # (from_stage, to_stage) -> this process's end of the edge connector
    while True:
        idle = not adapter.has_work()
        try:
            task = in_q.get(timeout=0.02) if idle else in_q.get_nowait()
        except queue.Empty:
            task = None
        except Exception:
            task = None
        drained = 0
        while task is not None:
            tt = task.get("type")
            if tt == OmniStageTaskType.SHUTDOWN:
                adapter.shutdown()
                out_q.put({"type": "stage_stopped", "stage_id": sid})
                return
            if tt == OmniStageTaskType.GENERATE:
                if paused:
                    held.append(task)
                else:
                    try:
                        _resolve_payload(task, edge_connectors)
                        adapter.add_task(task)
                    except Exception as e:
                        out_q.put({"request_id": task.get("request_id"), "stage_id": sid,
                                   "error": f"{type(e).__name__}: {e}", "error_tb": traceback.format_exc()})
            elif tt == OmniStageTaskType.UPDATE:
                if paused and any(t["request_id"] == task.get("request_id") for t in held):
                    held.append(task)           # keep it behind the request it belongs to
                else:
                    try:
                        adapter.update(task)
                    except Exception as e:
                        out_q.put({"request_id": task.get("request_id"), "stage_id": sid,
                                   "error": f"{type(e).__name__}: {e}", "error_tb": traceback.format_exc()})
            elif tt == OmniStageTaskType.ABORT:
                adapter.abort(list(task.get("request_ids") or [task.get("request_id")]))
                held = [t for t in held if t["request_id"] not in set(task.get("request_ids") or [task.get("request_id")])]
            elif tt == OmniStageTaskType.PROFILER_START:
                try:
                    adapter.start_profile(task.get("trace_dir"))
                except Exception as e:
                    logger.warning("stage %d: profiler start failed: %s", sid, e)
            elif tt == OmniStageTaskType.PROFILER_STOP:
                try:
                    out_q.put({"type": "profile", "stage_id": sid, "path": adapter.stop_profile()})
                except Exception as e:
                    logger.warning("stage %d: profiler stop failed: %s", sid, e)
            elif tt == OmniStageTaskType.PAUSE:
                paused = True
            elif tt == OmniStageTaskType.RESUME:
                paused = False
                for t in held:
                    if t.get("type") == OmniStageTaskType.UPDATE:
                        adapter.update(t)
                    else:
                        adapter.add_task(t)
                held = []
            drained += 1
            try:
                task = in_q.get_nowait() if drained < 256 else None
            except Exception:
                task = None
        if adapter.has_work():
            for r in adapter.step():
                out_q.put(r if in_process else to_host(r))       # queue messages between processes carry host data only


# =============================================================================== stage
class _RayWorkerHandle:
    """The slice of the Process API that ``OmniStage`` uses, over a Ray actor."""

    def __init__(self, actor):
        self.actor = actor
        self._dead = False

    def start(self):
        pass

    def is_alive(self) -> bool:
        return not self._dead

    def join(self, timeout=None):
        pass

    def terminate(self):
        from ..distributed import ray_utils
        ray_utils.kill_ray_actor(self.actor)
        self._dead = True


class OmniStage:
    def __init__(self, cfg: StageConfig, model: str | None, batch_timeout_s: float = 0.01,
                 stage_init_timeout: float = 300.0, worker_backend: str = "mp", placement_group=None):
        self.cfg = cfg
        self.worker_backend = worker_backend
        self._placement_group = placement_group
        self.stage_id = cfg.stage_id
        self.stage_type = cfg.stage_type
        self.model = model
        self.engine_args = cfg.engine_args
        self.model_stage = cfg.engine_args.get("model_stage")
        self.engine_input_source = list(cfg.engine_input_source)
        self.final_output = bool(cfg.final_output)
        self.final_output_type = cfg.final_output_type or ("image" if cfg.stage_type == "diffusion" else "text")
        self.is_comprehension = cfg.is_comprehension
        self.requires_multimodal_data = bool(cfg.runtime.get("requires_multimodal_data", False))
        self.custom_process_input_func = resolve_callable(cfg.custom_process_input_func)
        self.batch_timeout_s = batch_timeout_s
        self.stage_init_timeout = stage_init_timeout
        self.in_process = not bool(cfg.runtime.get("process", False))
        self.engine_outputs: Any = None
        self._in_q = self._out_q = None
        self._worker = None
        self._ready = False
        self._stopped = False

    # ------------------------------------------------------------------ lifecycle
    def init_stage_worker(self):
        if self.worker_backend == "ray":
            # one actor per stage, pinned to its placement-group bundle, running the same worker loop
            # over Ray queues (vllm_omni/distributed/ray_utils/utils.py:28-181)
            from ..distributed import ray_utils
            self.in_process = False
            self._in_q, self._out_q = ray_utils.make_queue(), ray_utils.make_queue()
            actor, _ = ray_utils.start_ray_actor(_stage_worker, self._placement_group, self.stage_id, self.cfg, self.model,
                                                 self._in_q, self._out_q, self.batch_timeout_s, False)
            self._worker = _RayWorkerHandle(actor)
            return
        if self.in_process:
            self._in_q, self._out_q = queue.Queue(), queue.Queue()
            self._worker = threading.Thread(target=_stage_worker, name=f"omni-stage-{self.stage_id}", daemon=True,
                                            args=(self.cfg, self.model, self._in_q, self._out_q, self.batch_timeout_s,
                                                  True))
        else:
            ctx = mp.get_context("spawn")
            self._in_q, self._out_q = ctx.Queue(), ctx.Queue()
            self._worker = ctx.Process(target=_stage_worker, name=f"omni-stage-{self.stage_id}", daemon=False,
                                       args=(self.cfg, self.model, self._in_q, self._out_q, self.batch_timeout_s,
                                             False))
        self._worker.start()

    def wait_ready(self, timeout: float | None = None) -> bool:
        timeout = self.stage_init_timeout if timeout is None else timeout
        deadline = time.monotonic() + timeout
        while time.monotonic() < deadline:
            try:
                msg = self._out_q.get(timeout=0.1)
            except Exception:
                if not self._worker.is_alive():
                    raise RuntimeError(f"stage {self.stage_id} worker exited during start-up")
                continue
            if msg.get("type") == "stage_ready":
                self._ready = True
                return True
            if msg.get("type") == "stage_error":
                raise RuntimeError(f"stage {self.stage_id} failed to start: {msg['error']}\n{msg.get('error_tb', '')}")
        return False

    def stop_stage_worker(self, join_timeout: float = 5.0):
        if self._worker is None or self._stopped:
            return
        self._stopped = True
        try:
            self._in_q.put({"type": OmniStageTaskType.SHUTDOWN})
        except Exception:
            pass
        self._worker.join(timeout=join_timeout)
        if self._worker.is_alive() and not self.in_process:
            self._worker.terminate()

    def check_health(self) -> bool:
        return self._worker is not None and self._worker.is_alive()

    # ------------------------------------------------------------------ traffic
    def submit(self, task: dict) -> None:
        task.setdefault("type", OmniStageTaskType.GENERATE)
        task.setdefault("submit_ts", time.time())
        self._in_q.put(task if self.in_process else to_host(task))

    def try_collect(self) -> dict | None:
        try:
            return self._out_q.get_nowait()
        except Exception:
            return None

    def abort(self, request_ids: list[str]):
        self._in_q.put({"type": OmniStageTaskType.ABORT, "request_ids": list(request_ids)})

    def pause(self):
        self._in_q.put({"type": OmniStageTaskType.PAUSE})

    def resume(self):
        self._in_q.put({"type": OmniStageTaskType.RESUME})

    def start_profile(self, trace_dir=None):
        self._in_q.put({"type": OmniStageTaskType.PROFILER_START, "trace_dir": trace_dir})

    def stop_profile(self):
        self._in_q.put({"type": OmniStageTaskType.PROFILER_STOP})

    def set_engine_outputs(self, outs) -> None:
        self.engine_outputs = outs

    def default_sampling_params(self):
        d = dict(self.cfg.default_sampling_params or {})
        if self.stage_type == "diffusion":
            names = OmniDiffusionSamplingParams.__dataclass_fields__
            return OmniDiffusionSamplingParams(**{k: v for k, v in d.items() if k in names})
        names = SamplingParams.__dataclass_fields__
        return SamplingParams(**{k: v for k, v in d.items() if k in names})

    # ------------------------------------------------------------------ inputs from upstream
    def process_engine_inputs(self, stage_list: list["OmniStage"], prompt=None) -> list:
        """Inputs of this stage from its upstream stages' latest outputs
        (vllm_omni/entrypoints/omni_stage.py:585-633)."""
        if self.custom_process_input_func is not None:
            return self.custom_process_input_func(stage_list, self.engine_input_source, prompt,
                                                  self.requires_multimodal_data)
        if not self.engine_input_source:
            raise ValueError("engine_input_source is empty")
        src = stage_list[self.engine_input_source[0]].engine_outputs
        prompts = prompt if isinstance(prompt, list) else [prompt]
        outs = []
        for i, so in enumerate(src):
            ro = getattr(so, "request_output", None) or so
            p = prompts[i] if i < len(prompts) else None
            mm = p.get("multi_modal_data") if (isinstance(p, dict) and self.requires_multimodal_data) else None
            ti = OmniTokensPrompt(prompt_token_ids=list(ro.outputs[0].token_ids))
            if mm is not None:
                ti["multi_modal_data"] = mm
            outs.append(ti)
        return outs


# ================================================================================ build
def _default_diffusion_stage(kwargs: dict) -> dict:
    pc = kwargs.get("parallel_config")
    world = pc.world_size if hasattr(pc, "world_size") else 1
    return {"stage_id": 0, "stage_type": "diffusion",
            "runtime": {"process": False, "devices": ",".join(str(i) for i in range(world)), "max_batch_size":
                        int(kwargs.get("max_batch_size", 1))},
            "engine_args": {**kwargs, "model_stage": "diffusion"}, "final_output": True,
            "final_output_type": "image"}


def build_stages(model, stage_configs_path, kwargs: dict, stage_init_timeout=300, shm_threshold_bytes=65536,
                 worker_backend="mp", batch_timeout=10):
    """Returns (stages, connectors, pipeline_config).  ``batch_timeout`` is in milliseconds."""
    from ..connectors.factory import initialize_orchestrator_connectors
    placement_group = None
    if worker_backend == "ray":
        from ..distributed import ray_utils
        ray_utils.initialize_ray_cluster()
    path = stage_configs_path or resolve_model_config_path(model)
    if path is not None:
        base = {k: v for k, v in kwargs.items() if k in ("dtype", "seed", "device", "load_format")}
        pcfg = load_stage_configs_from_yaml(path, base)
    else:
        from .utils import load_stage_configs_from_dict
        pcfg = load_stage_configs_from_dict({"stage_args": []})
        pcfg.stages = [StageConfig.from_dict(_default_diffusion_stage(dict(kwargs)))]
    inject_omni_kv_config(pcfg.stages)
    if worker_backend == "ray":
        placement_group = ray_utils.create_placement_group(pcfg.stages)
        shm_threshold_bytes = ray_utils.SHM_THRESHOLD_UNDER_RAY     # payloads ride on the Ray queues
    connectors = initialize_orchestrator_connectors(pcfg.stages, pcfg.runtime, shm_threshold_bytes=shm_threshold_bytes)
    stages = [OmniStage(sc, model, batch_timeout_s=batch_timeout / 1000.0, stage_init_timeout=stage_init_timeout,
                        worker_backend=worker_backend, placement_group=placement_group)
              for sc in pcfg.stages]
    for s in stages:
        s.init_stage_worker()
    for s in stages:
        if not s.wait_ready():
            logger.warning("stage %d not ready after %ss", s.stage_id, stage_init_timeout)
    return stages, connectors, pcfg
