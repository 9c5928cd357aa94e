"""Blocking multi-stage generation loop used by ``Omni.generate``.

Mirrors ``_run_generation`` of the reference (vllm_omni/entrypoints/omni.py:640-910): seed
stage 0 with every request, then poll the stages; when a stage finishes a request its
outputs become the input of every stage that lists it in ``engine_input_source`` (through
that stage's input processor and the edge's connector); outputs of stages marked
``final_output`` are returned to the caller in request order.
"""
from __future__ import annotations

import time
from typing import Any

from ..logger import init_logger
from ..outputs import OmniRequestOutput, RequestOutput
from .stage_utils import OmniStageTaskType

logger = init_logger(__name__)


class StageError(RuntimeError):
    def __init__(self, stage_id, request_id, error, tb=""):
        super().__init__(f"stage {stage_id} failed on request {request_id}: {error}\n{tb}")
        self.stage_id, self.request_id = stage_id, request_id


def wrap_stage_output(stage, out) -> OmniRequestOutput:
    if isinstance(out, OmniRequestOutput):
        out.stage_id = stage.stage_id if out.stage_id is None else out.stage_id
        return out
    if isinstance(out, RequestOutput):
        return OmniRequestOutput.from_pipeline(stage.stage_id, stage.final_output_type, out)
    raise TypeError(f"unexpected stage output {type(out)!r}")


def send_downstream(omni, src_stage, dst_stage, request_id: str, prompt, sampling_params, mark: dict | None = None) -> None:
    """Build the next stage's inputs from ``src_stage.engine_outputs`` and submit them,
    moving the payload through the edge connector (connectors/adapter.py).  ``mark`` is merged into the
    ``additional_information`` of every input (e.g. "the producer is still running")."""
    from ..connectors.adapter import try_send_via_connector
    inputs = dst_stage.process_engine_inputs(omni.stage_list, prompt)
    if mark:
        for it in (inputs if isinstance(inputs, list) else [inputs]):
            if isinstance(it, dict):
                it.setdefault("additional_information", {}).update(mark)
    connector = omni.connectors.get((src_stage.stage_id, dst_stage.stage_id))
    task = {"type": OmniStageTaskType.GENERATE, "request_id": request_id, "sampling_params": sampling_params,
            "from_stage": src_stage.stage_id}
    sent = False
    if connector is not None and not dst_stage.in_process:
        sent = try_send_via_connector(connector, src_stage.stage_id, dst_stage.stage_id, request_id, inputs, task,
                                      omni.metrics)
        if sent:
            # the receiving process opens its own end of the edge from this description
            spec = getattr(connector, "spec", None)
            task["connector_meta"]["spec"] = spec or {"name": type(connector).__name__, "extra": dict(connector.config)}
    if not sent:
        task["engine_inputs"] = inputs
    dst_stage.submit(task)


def run_generation(omni, prompts: list, sampling_params_list: list, request_ids: list[str],
                   poll_interval_s: float = 0.0005, timeout_s: float | None = None) -> list[OmniRequestOutput]:
    stages = omni.stage_list
    n_stage = len(stages)
    prompt_of = dict(zip(request_ids, prompts))
    consumers = {s.stage_id: [d for d in stages if s.stage_id in d.engine_input_source] for s in stages}
    final_stages = [s.stage_id for s in stages if s.final_output] or [stages[-1].stage_id]
    # a request is complete when every final stage and every leaf stage has reported it
    must_finish = set(final_stages) | {s.stage_id for s in stages if not consumers[s.stage_id]}
    done: dict[str, set] = {r: set() for r in request_ids}
    results: dict[str, list[OmniRequestOutput]] = {r: [] for r in request_ids}
    t_start = time.time()
    for rid, p in zip(request_ids, prompts):
        omni.metrics.on_request_start(rid, t_start)
        stages[0].submit({"type": OmniStageTaskType.GENERATE, "request_id": rid, "engine_inputs": p,
                          "sampling_params": sampling_params_list[0]})
    remaining = set(request_ids)
    deadline = None if timeout_s is None else time.monotonic() + timeout_s
    while remaining:
        progressed = False
        for stage in stages:
            res = stage.try_collect()
            if res is None:
                continue
            progressed = True
            if res.get("type") in ("profile", "stage_stopped", "stage_ready"):
                continue
            rid = res.get("request_id")
            if "error" in res:
                for s in stages:
                    s.abort([r for r in remaining])
                raise StageError(stage.stage_id, rid, res["error"], res.get("error_tb", ""))
            if rid not in remaining:
                continue
            outs = res.get("engine_outputs")
            if not res.get("finished", True):
                continue                       # streaming partials are for AsyncOmni
            outs = outs if isinstance(outs, list) else [outs]
            stage.set_engine_outputs(outs)
            if "metrics" in res:
                omni.metrics.on_stage_metrics(stage.stage_id, rid, res["metrics"])
            if stage.stage_id in final_stages:
                for o in outs:
                    w = wrap_stage_output(stage, o)
                    w.request_id = w.request_id or rid
                    w.final_output_type = stage.final_output_type if w.is_pipeline_output else w.final_output_type
                    results[rid].append(w)
            for dst in consumers[stage.stage_id]:
                send_downstream(omni, stage, dst, rid, prompt_of[rid], sampling_params_list[dst.stage_id])
            done[rid].add(stage.stage_id)
            if must_finish <= done[rid]:
                remaining.discard(rid)
                omni.metrics.on_finalize_request(rid)
        if not progressed:
            for s in stages:
                if not s.check_health():
                    raise StageError(s.stage_id, None, "stage worker is not alive")
            if deadline is not None and time.monotonic() > deadline:
                raise TimeoutError(f"generation timed out after {timeout_s}s; unfinished: {sorted(remaining)}")
            time.sleep(poll_interval_s)
    out: list[OmniRequestOutput] = []
    for rid in request_ids:
        out.extend(results[rid])
    return out
