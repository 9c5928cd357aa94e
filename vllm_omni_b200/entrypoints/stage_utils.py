"""Helpers shared by the stage workers: task types, device pinning, IPC payload hand-off,
JSONL logging (vllm_omni/entrypoints/stage_utils.py)."""
from __future__ import annotations

import enum
import json
import os
from typing import Any


class OmniStageTaskType(enum.Enum):
    GENERATE = "generate"
    ABORT = "abort"
    SHUTDOWN = "shutdown"
    PROFILER_START = "profiler_start"
    PROFILER_STOP = "profiler_stop"
    PAUSE = "pause"
    RESUME = "resume"


SHUTDOWN_TASK = {"type": OmniStageTaskType.SHUTDOWN}


def is_profiler_task(t: OmniStageTaskType) -> bool:
    return t in (OmniStageTaskType.PROFILER_START, OmniStageTaskType.PROFILER_STOP)


def parse_devices(devices) -> list[int] | None:
    if devices is None or devices == "cpu" or devices == "":
        return None
    if isinstance(devices, int):
        return [devices]
    return [int(x) for x in str(devices).split(",") if x.strip() != ""]


def set_stage_devices(stage_id: int, devices, in_process: bool = False) -> list[int] | None:
    """Pin a stage to its GPUs.  ``devices`` are logical indices into the current
    ``CUDA_VISIBLE_DEVICES``.  A stage in its own process rewrites the variable (before CUDA is
    initialised) so that its first device is ``cuda:0``; an in-process stage cannot do that and
    gets the list of physical ordinals to pass to its engine instead."""
    want = parse_devices(devices)
    if want is None:
        return None
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    mapping = [x.strip() for x in vis.split(",")] if vis else None
    if in_process:
        return want
    phys = [mapping[i] if mapping and i < len(mapping) else str(i) for i in want]
    os.environ["CUDA_VISIBLE_DEVICES"] = ",".join(phys)
    return list(range(len(phys)))


def append_jsonl(path: str | None, record: dict) -> None:
    if not path:
        return
    with open(path, "a") as f:
        f.write(json.dumps(record, default=str) + "\n")


def maybe_dump_to_ipc(obj: Any, connector, stage_id: int, key: str):
    """Large results leave the stage process through the connector; the queue carries the
    descriptor only."""
    ok, size, meta = connector.put(stage_id, "orch", key, obj)
    if not ok:
        raise RuntimeError(f"stage {stage_id}: could not export result {key}")
    return {"ipc_meta": meta, "size": size}


def maybe_load_from_ipc(desc: dict, connector, stage_id: int, key: str):
    res = connector.get(stage_id, "orch", key, desc["ipc_meta"])
    if res is None:
        raise RuntimeError(f"stage {stage_id}: result {key} never arrived")
    return res[0]
