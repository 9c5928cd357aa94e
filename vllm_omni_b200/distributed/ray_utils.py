"""Ray worker backend for stages (vllm_omni/distributed/ray_utils/utils.py:28-181).

One Ray actor per stage runs the same ``_stage_worker`` loop that the process backend runs in a
spawned process; a placement group reserves one bundle per stage with that stage's GPU count,
and the stage's in/out queues are Ray queues.  Under Ray the shared-memory threshold is
infinite (payloads ride on the queue / object store).  Ray is an optional dependency: every
entry point calls ``require_ray`` first and fails with a clear message when it is absent.
"""
from __future__ import annotations

import sys
from typing import Any


def ray_available() -> bool:
    try:
        import ray  # noqa: F401
        return True
    except Exception:  # noqa: BLE001
        return False


def require_ray():
    if not ray_available():
        raise RuntimeError("worker_backend='ray' needs the `ray` package, which is not installed here; "
                           "use worker_backend='mp' (one process per stage) instead")
    import ray
    return ray


SHM_THRESHOLD_UNDER_RAY = sys.maxsize


def initialize_ray_cluster(address: str | None = None, num_gpus: int | None = None):
    ray = require_ray()
    if not ray.is_initialized():
        ray.init(address=address, num_gpus=num_gpus, ignore_reinit_error=True)
    return ray


def stage_bundles(stage_configs) -> list[dict[str, float]]:
    """One placement-group bundle per stage: its GPU count (from ``runtime.devices``) and a CPU."""
    out = []
    for sc in stage_configs:
        devs = str((sc.runtime or {}).get("devices", "0"))
        n = len([d for d in devs.split(",") if d.strip() != ""])
        out.append({"GPU": float(max(1, n)), "CPU": 1.0})
    return out


def create_placement_group(stage_configs, strategy: str = "PACK"):
    ray = require_ray()
    from ray.util.placement_group import placement_group
    pg = placement_group(stage_bundles(stage_configs), strategy=strategy)
    ray.get(pg.ready())
    return pg


def start_ray_actor(worker_fn, placement_group, bundle_index: int, *args: Any, **kwargs: Any):
    """Run ``worker_fn(*args, **kwargs)`` inside an actor pinned to one bundle."""
    ray = require_ray()
    from ray.util.scheduling_strategies import PlacementGroupSchedulingStrategy

    @ray.remote
    class _StageActor:
        def run(self, fn, a, kw):
            return fn(*a, **kw)

    bundle = placement_group.bundle_specs[bundle_index]
    actor = _StageActor.options(
        num_gpus=bundle.get("GPU", 0), num_cpus=bundle.get("CPU", 1),
        scheduling_strategy=PlacementGroupSchedulingStrategy(placement_group=placement_group,
                                                             placement_group_bundle_index=bundle_index)).remote()
    return actor, actor.run.remote(worker_fn, args, kwargs)


def make_queue(maxsize: int = 0):
    require_ray()
    from ray.util.queue import Queue
    return Queue(maxsize=maxsize)


def kill_ray_actor(actor) -> None:
    ray = require_ray()
    try:
        ray.kill(actor)
    except Exception:  # noqa: BLE001
        pass
