"""ctypes loader for the in-tree CUDA libraries.

On a machine with a GPU a missing library is an error: the CUDA path is the product and
there is no silent eager fallback.  On CPU-only machines the ops fall back to their
PyTorch reference implementations so that the host-side logic stays testable.
"""
from __future__ import annotations

import ctypes
import os
import functools
from pathlib import Path

import torch

from ..build import lib_path


class NativeError(RuntimeError):
    pass


# kernels launched per exported entry point (default 1); used for the launch counter
_KERNELS_PER_CALL = {"omni_rel_l1": 2, "omni_rel_l1_parts": 0, "omni_paged_decode": 2, "omni_gemm_set_pair_mode": 0}
launch_count = 0
_timing: list | None = None      # (entry point, start event, stop event) while kernel timing is on


def enable_kernel_timing(on: bool = True) -> None:
    """Bracket every native launch with CUDA events; read the result with ``kernel_timing_summary``."""
    global _timing
    _timing = [] if on else None


def kernel_timing_summary(reset: bool = True) -> dict[str, dict]:
    """Per entry point: launches, total and mean device time in ms (synchronises the device)."""
    global _timing
    out: dict[str, dict] = {}
    if not _timing:
        return out
    torch.cuda.synchronize()
    for name, e0, e1 in _timing:
        d = out.setdefault(name, {"launches": 0, "total_ms": 0.0})
        d["launches"] += 1
        d["total_ms"] += e0.elapsed_time(e1)
    for d in out.values():
        d["mean_us"] = 1000.0 * d["total_ms"] / max(1, d["launches"])
    if reset:
        _timing = []
    return out


class _CountingLib:
    """CDLL proxy that counts the kernel launches made through it."""

    def __init__(self, cdll: ctypes.CDLL):
        self._cdll = cdll
        self._fns: dict = {}

    def __getattr__(self, name):
        fn = self._fns.get(name)
        if fn is None:
            raw = getattr(self._cdll, name)
            n = _KERNELS_PER_CALL.get(name, 1)

            def fn(*args, _raw=raw, _n=n, _name=name):
                global launch_count
                launch_count += _n
                if _timing is not None and _n:
                    # device timers around the launch (CUDA events on the launching stream); only
                    # meaningful outside CUDA-graph capture
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    rc = _raw(*args)
                    e1.record()
                    _timing.append((_name, e0, e1))
                    return rc
                return _raw(*args)

            self._fns[name] = fn
        return fn


def bounds_check_enabled() -> bool:
    """``OMNI_BOUNDS_CHECK=1``: load the checked twins (built with -DOMNI_BOUNDS_CHECK) of the libraries
    that have one; their kernels test index operands against the limits the wrappers pass and report
    ``ERR_BOUNDS`` through the status word instead of touching memory outside a buffer."""
    return os.environ.get("OMNI_BOUNDS_CHECK", "0") == "1"


@functools.lru_cache(maxsize=None)
def lib(name: str) -> _CountingLib:
    p: Path = lib_path(name)
    if bounds_check_enabled():
        twin = lib_path(name, checked=True)
        if twin.exists():
            p = twin
    if not p.exists():
        raise NativeError(
            f"{p} is missing: run `python -m vllm_omni_b200.build` (nvcc, sm_100a) before using the GPU ops")
    return _CountingLib(ctypes.CDLL(str(p)))


def have_gpu() -> bool:
    return torch.cuda.is_available()


_status: dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 that kernels set when one of their bounded waits ran out."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = t
    return t


def check_status(device: torch.device | None = None) -> int:
    """Read (and clear) the status word; raises if a kernel reported a timeout."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    t = status_word(device)
    v = int(t.item())
    if v != 0:
        t.zero_()
        raise NativeError(f"a kernel reported error status {v} (bounded wait ran out)")
    return v


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def check_rc(rc: int, what: str) -> None:
    if rc != 0:
        raise NativeError(f"{what} failed with code {rc}")
