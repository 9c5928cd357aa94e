"""Python face of the lock-free shared-memory ring in ``csrc/rt_host.cpp``: a single-producer /
single-consumer queue of byte messages between two processes (fixed-size slots, sequence
counters, no locks, no syscalls on the data path).  It plays the role of vLLM's shm
``MessageQueue`` that the reference uses between the diffusion engine and its workers
(vllm_omni/diffusion/scheduler.py)."""
from __future__ import annotations

import ctypes
import pickle
import time
from typing import Any

from ..ops import _native as nv


def _lib():
    from ..build import build_one, lib_path
    if not lib_path("rt_host").exists():        # host-only C++: build on first use where the tree is fresh
        build_one("rt_host")
    lib = nv.lib("rt_host")._cdll
    if not getattr(lib, "_ring_typed", False):
        lib.omni_ring_open.restype = ctypes.c_void_p
        lib.omni_ring_open.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_uint32, ctypes.c_uint32]
        lib.omni_ring_close.argtypes = [ctypes.c_void_p]
        lib.omni_ring_push.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_uint32]
        lib.omni_ring_pop.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32]
        lib.omni_ring_size.argtypes = [ctypes.c_void_p]
        lib.omni_ring_slot_bytes.argtypes = [ctypes.c_void_p]
        lib.omni_ring_slot_bytes.restype = ctypes.c_uint32
        lib._ring_typed = True
    return lib


class ShmRing:
    def __init__(self, name: str, create: bool = False, slot_bytes: int = 65536, num_slots: int = 64):
        self._lib = _lib()
        self.name = name if name.startswith("/") else "/" + name
        self._h = self._lib.omni_ring_open(self.name.encode(), 1 if create else 0, slot_bytes, num_slots)
        if not self._h:
            raise OSError(f"cannot {'create' if create else 'attach to'} shared-memory ring {self.name}")
        self.max_message = int(self._lib.omni_ring_slot_bytes(self._h))
        self._buf = ctypes.create_string_buffer(self.max_message)

    def push(self, msg: bytes, timeout: float | None = 0.0) -> bool:
        """False when the ring stayed full for ``timeout`` seconds (None = wait forever)."""
        if len(msg) > self.max_message:
            raise ValueError(f"message of {len(msg)} bytes exceeds the slot size {self.max_message}")
        t0 = time.monotonic()
        while True:
            rc = self._lib.omni_ring_push(self._h, msg, len(msg))
            if rc == 0:
                return True
            if timeout is not None and time.monotonic() - t0 >= timeout:
                return False
            time.sleep(0.0002)

    def pop(self, timeout: float | None = 0.0) -> bytes | None:
        t0 = time.monotonic()
        while True:
            n = self._lib.omni_ring_pop(self._h, self._buf, self.max_message)
            if n >= 0:
                return self._buf.raw[:n]
            if timeout is not None and time.monotonic() - t0 >= timeout:
                return None
            time.sleep(0.0002)

    def put_obj(self, obj: Any, timeout: float | None = None) -> bool:
        return self.push(pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL), timeout)

    def get_obj(self, timeout: float | None = None) -> Any:
        b = self.pop(timeout)
        return None if b is None else pickle.loads(b)

    def __len__(self) -> int:
        return int(self._lib.omni_ring_size(self._h))

    def close(self) -> None:
        if self._h:
            self._lib.omni_ring_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass
