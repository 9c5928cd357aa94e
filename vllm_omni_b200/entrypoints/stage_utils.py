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
    UPDATE = "update"          # late input for a running request (rows of an upstream stage that is still generating)


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


def to_host(obj, _seen=None):
    """Move every CUDA tensor inside a message (dicts, lists, tuples, plain objects) to host memory, in place
    where the container allows it.  Messages between the orchestrator and a stage PROCESS travel through
    ``multiprocessing`` queues: a CUDA tensor in them becomes a CUDA-IPC handle whose memory the producer must
    keep alive, which the receiver cannot pass on to a third process ("Attempted to send CUDA tensor received
    from another process") and which costs a handle per tensor.  Device payloads have their own path (the
    device connector); everything on the queues is host data."""
    import torch
    if isinstance(obj, torch.Tensor):
        return obj.detach().cpu() if obj.is_cuda else obj
    if obj is None or isinstance(obj, (str, bytes, int, float, bool)):
        return obj
    _seen = set() if _seen is None else _seen
    if id(obj) in _seen:
        return obj
    _seen.add(id(obj))
    if isinstance(obj, dict):
        for k in list(obj):
            obj[k] = to_host(obj[k], _seen)
        return obj
    if isinstance(obj, list):
        for i in range(len(obj)):
            obj[i] = to_host(obj[i], _seen)
        return obj
    if isinstance(obj, tuple):
        return type(obj)(to_host(v, _seen) for v in obj) if type(obj) is tuple else obj
    d = getattr(obj, "__dict__", None)
    if isinstance(d, dict) and not isinstance(obj, type) and type(obj).__module__.startswith("vllm_omni_b200"):
        for k in list(d):
            try:
                setattr(obj, k, to_host(d[k], _seen))
            except Exception:   # noqa: BLE001  (read-only attribute)
                pass
    return obj
