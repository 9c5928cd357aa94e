"""torch.profiler wrapper with the reference's trace naming
(vllm_omni/diffusion/profiler/torch_profiler.py: chrome trace ``{template}_rank{N}.json``,
gzip in a background thread; directory from ``VLLM_TORCH_PROFILER_DIR``) plus NVTX ranges
for nsight-style tools."""
from __future__ import annotations

import gzip
import os
import shutil
import threading
import time
from contextlib import contextmanager

import torch


class TorchProfiler:
    def __init__(self, trace_dir: str | None = None, rank: int | None = None, template: str = "omni_trace"):
        self.trace_dir = trace_dir or os.environ.get("VLLM_TORCH_PROFILER_DIR") or os.environ.get("OMNI_PROFILER_DIR")
        if not self.trace_dir:
            raise RuntimeError("set VLLM_TORCH_PROFILER_DIR (or pass trace_dir) to enable profiling")
        self.rank = int(os.environ.get("RANK", "0")) if rank is None else rank
        self.template = template
        self._prof = None

    def start(self):
        os.makedirs(self.trace_dir, exist_ok=True)
        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        self._prof = torch.profiler.profile(activities=acts, record_shapes=True, profile_memory=True, with_stack=False)
        self._prof.__enter__()

    def stop(self) -> str:
        self._prof.__exit__(None, None, None)
        path = os.path.join(self.trace_dir, f"{self.template}_{int(time.time())}_rank{self.rank}.json")
        self._prof.export_chrome_trace(path)
        self._prof = None

        def _gz():
            with open(path, "rb") as fi, gzip.open(path + ".gz", "wb") as fo:
                shutil.copyfileobj(fi, fo)
            os.remove(path)
        threading.Thread(target=_gz, daemon=True).start()
        return path + ".gz"


@contextmanager
def nvtx_range(name: str):
    """NVTX range on GPU builds, no-op elsewhere."""
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()
