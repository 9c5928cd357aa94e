"""Paged KV cache bookkeeping: block pool (C++ allocator in csrc/rt_host.cpp, Python fallback)
and the per-request block tables.  The device tensors themselves belong to the model runner;
this class only decides which pages a request owns."""
from __future__ import annotations

import ctypes

from ..build import lib_path


class BlockPool:
    def __init__(self, num_blocks: int):
        self.num_blocks = num_blocks
        self._lib = None
        p = lib_path("rt_host")
        if p.exists():
            lib = ctypes.CDLL(str(p))
            lib.omni_balloc_create.restype = ctypes.c_void_p
            lib.omni_balloc_create.argtypes = [ctypes.c_int]
            for fn in ("omni_balloc_destroy", "omni_balloc_num_free", "omni_balloc_alloc", "omni_balloc_ref",
                       "omni_balloc_free"):
                getattr(lib, fn).argtypes = {"omni_balloc_destroy": [ctypes.c_void_p],
                                             "omni_balloc_num_free": [ctypes.c_void_p],
                                             "omni_balloc_alloc": [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p],
                                             "omni_balloc_ref": [ctypes.c_void_p, ctypes.c_int],
                                             "omni_balloc_free": [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]}[fn]
            self._lib = lib
            self._h = lib.omni_balloc_create(num_blocks)
        else:  # pure-Python twin with the same semantics
            self._free = list(range(num_blocks - 1, -1, -1))
            self._ref = [0] * num_blocks

    @property
    def num_free(self) -> int:
        return self._lib.omni_balloc_num_free(self._h) if self._lib else len(self._free)

    def alloc(self, n: int) -> list[int] | None:
        if n == 0:
            return []
        if self._lib:
            out = (ctypes.c_int32 * n)()
            return list(out) if self._lib.omni_balloc_alloc(self._h, n, out) == 0 else None
        if len(self._free) < n:
            return None
        out = [self._free.pop() for _ in range(n)]
        for b in out:
            self._ref[b] = 1
        return out

    def ref(self, block: int) -> int:
        if self._lib:
            return self._lib.omni_balloc_ref(self._h, block)
        if self._ref[block] <= 0:
            return -1
        self._ref[block] += 1
        return self._ref[block]

    def free(self, blocks: list[int]) -> int:
        if not blocks:
            return 0
        if self._lib:
            arr = (ctypes.c_int32 * len(blocks))(*blocks)
            r = self._lib.omni_balloc_free(self._h, len(blocks), arr)
        else:
            r = 0
            for b in blocks:
                if self._ref[b] <= 0:
                    r = -1
                    break
                self._ref[b] -= 1
                if self._ref[b] == 0:
                    self._free.append(b)
                    r += 1
        if r < 0:
            raise RuntimeError("double free of a KV block")
        return r

    def __del__(self):
        if getattr(self, "_lib", None) is not None:
            try:
                self._lib.omni_balloc_destroy(self._h)
            except Exception:
                pass


class KVCacheManager:
    def __init__(self, num_blocks: int, block_size: int):
        self.block_size = block_size
        self.pool = BlockPool(num_blocks)

    def blocks_needed(self, request, num_new_tokens: int) -> int:
        total = request.num_computed_tokens + num_new_tokens
        need = (total + self.block_size - 1) // self.block_size
        return max(0, need - len(request.block_ids))

    def allocate_slots(self, request, num_new_tokens: int) -> bool:
        """Make sure ``request`` owns pages for its next ``num_new_tokens`` tokens."""
        n = self.blocks_needed(request, num_new_tokens)
        if n == 0:
            return True
        got = self.pool.alloc(n)
        if got is None:
            return False
        request.block_ids.extend(got)
        return True

    def slot_mapping(self, request, start: int, n: int) -> list[int]:
        bs = self.block_size
        return [request.block_ids[t // bs] * bs + t % bs for t in range(start, start + n)]

    def free(self, request) -> None:
        self.pool.free(request.block_ids)
        request.block_ids = []

    @property
    def usage(self) -> float:
        return 1.0 - self.pool.num_free / max(1, self.pool.num_blocks)
