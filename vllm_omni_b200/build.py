"""In-tree build of the sm_100a CUDA libraries.

Every ``csrc/*.cu`` becomes ``_lib/libomni_<name>.so`` with a plain C ABI that
``vllm_omni_b200.ops`` loads through ctypes.  nvcc cross-compiles without a GPU, so the
build runs on CPU-only machines; the resulting libraries are only loaded where a GPU is
present.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "_lib"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-pthread"]
# libraries that also get a checked twin (-DOMNI_BOUNDS_CHECK, ``libomni_<name>_checked.so``): kernels that take
# addresses from index operands test them and report through the status word instead of faulting;
# ``OMNI_BOUNDS_CHECK=1`` makes ``ops/_native.lib`` load the twin
CHECKED = ("kv_cache", "moe")


def lib_path(name: str, checked: bool = False) -> Path:
    return LIB / f"libomni_{name}{'_checked' if checked else ''}.so"


def _newest_header_mtime() -> float:
    hs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    return max((h.stat().st_mtime for h in hs), default=0.0)


def _compile(src: Path, force: bool, checked: bool = False) -> str:
    out = lib_path(src.stem, checked)
    dep_m = max(src.stat().st_mtime, _newest_header_mtime())
    if not force and out.exists() and out.stat().st_mtime >= dep_m:
        return f"up-to-date {out.name}"
    if src.suffix == ".cu":
        nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
        cmd = [nvcc, *NVCC_FLAGS, *(["-DOMNI_BOUNDS_CHECK"] if checked else []), "-I", str(CSRC), "-o", str(out), str(src)]
    else:
        cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")     # NVTX v3 headers
        inc = ["-I", cuda_inc] if os.path.isdir(cuda_inc) else []
        cmd = [os.environ.get("CXX", "g++"), *CXX_FLAGS, "-I", str(CSRC), *inc, "-o", str(out), str(src), "-lrt", "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"build failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    return f"built {out.name}"


def build_all(force: bool = False, verbose: bool = True) -> list[str]:
    LIB.mkdir(exist_ok=True)
    srcs = sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cpp"))
    jobs = [(s, False) for s in srcs] + [(s, True) for s in srcs if s.stem in CHECKED]
    with ThreadPoolExecutor(max_workers=min(8, len(jobs) or 1)) as ex:
        msgs = list(ex.map(lambda j: _compile(j[0], force, j[1]), jobs))
    if verbose:
        for m in msgs:
            print("[build]", m)
    return msgs


def build_one(name: str, force: bool = False) -> str:
    """Build a single library by source stem (e.g. ``"rt_host"``): the host-only pieces compile in a
    second with g++ and are needed by CPU-side code paths too."""
    LIB.mkdir(exist_ok=True)
    for ext in (".cu", ".cpp"):
        src = CSRC / f"{name}{ext}"
        if src.exists():
            return _compile(src, force)
    raise FileNotFoundError(f"no source for library {name!r} under {CSRC}")


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
