"""Per-process GPU memory accounting for stages that share a GPU
(vllm_omni/worker/gpu_memory_utils.py:22-124, worker/base.py:24-108).

``gpu_memory_utilization`` is a share of the WHOLE device granted to one stage.  When several
stages initialise on the same GPU at once, "free memory" is a moving target, so the KV-cache
budget of a stage is computed from what THIS process holds (NVML's per-PID figure):

    kv_budget = total * utilization - memory_of_this_process

Only reads NVML; nothing here changes a device setting.  NVML handles come from ``pynvml`` when
present; the functions take the module as a parameter so that tests pass a fake.
"""
from __future__ import annotations

import os


def _nvml():
    try:
        import pynvml
        return pynvml
    except Exception:  # noqa: BLE001
        return None


def parse_cuda_visible_devices() -> list:
    """CUDA_VISIBLE_DEVICES as a list of physical indices (int) or UUID / MIG ids (str)."""
    out = []
    for item in os.environ.get("CUDA_VISIBLE_DEVICES", "").split(","):
        item = item.strip()
        if not item:
            continue
        try:
            out.append(int(item))
        except ValueError:
            out.append(item)
    return out


def physical_device(local_index: int):
    vis = parse_cuda_visible_devices()
    if not vis:
        return local_index
    if local_index >= len(vis):
        raise IndexError(f"local device {local_index} is outside CUDA_VISIBLE_DEVICES ({vis})")
    return vis[local_index]


def process_gpu_memory(local_index: int = 0, pid: int | None = None, nvml=None) -> int | None:
    """Bytes of device memory held by ``pid`` (default: this process) on the device, or None when
    NVML is unavailable or does not list the process (e.g. another PID namespace)."""
    nvml = nvml or _nvml()
    if nvml is None:
        return None
    pid = os.getpid() if pid is None else pid
    try:
        nvml.nvmlInit()
    except Exception:  # noqa: BLE001
        return None
    try:
        dev = physical_device(local_index)
        h = nvml.nvmlDeviceGetHandleByUUID(dev) if isinstance(dev, str) else nvml.nvmlDeviceGetHandleByIndex(dev)
        for p in nvml.nvmlDeviceGetComputeRunningProcesses(h):
            if p.pid == pid:
                return int(p.usedGpuMemory or 0)
        return None
    except Exception:  # noqa: BLE001
        return None
    finally:
        try:
            nvml.nvmlShutdown()
        except Exception:  # noqa: BLE001
            pass


def kv_cache_budget(total_bytes: int, free_bytes: int, utilization: float, local_index: int = 0, nvml=None,
                    pid: int | None = None) -> int:
    """Bytes this stage may still take for its KV cache.

    With NVML's per-process figure: ``total * utilization - own usage``, additionally capped by
    what is free right now.  Without it: the classic ``free - total * (1 - utilization)``."""
    own = process_gpu_memory(local_index, pid=pid, nvml=nvml)
    if own is None:
        return max(0, int(free_bytes - total_bytes * (1.0 - utilization)))
    return max(0, min(int(total_bytes * utilization) - own, int(free_bytes)))
