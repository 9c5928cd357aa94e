"""Symmetric peer-memory arenas for the fused compute+collective kernels.

Every rank of a group allocates an arena of the same size (``cudaMalloc`` in
csrc/peer_rt.cu), exports it as a CUDA IPC handle, and maps all peers' arenas, which makes a
peer's memory addressable by ordinary loads and stores inside our kernels (NVLink / NVSwitch
P2P).  Tensors are carved from the arena with a bump allocator, in the same order on every
rank, so the i-th allocation sits at the same offset everywhere ("symmetric").  A flag page
plus a device-resident epoch counter implement the bounded-wait barrier.

The reference has no such layer: all of its cross-GPU traffic is NCCL calls issued between
kernels (vllm_omni/diffusion/distributed/group_coordinator.py).
"""
from __future__ import annotations

import ctypes
import os

import torch

from ..ops import _native as nv

_CANARY_BYTE = 0xA5
_ALIGN = 1024


class _DevMem:
    """Exposes a raw device pointer to torch through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int, owner=None):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}
        self._owner = owner


def tensor_from_ptr(ptr: int, shape, dtype: torch.dtype, device: torch.device, owner=None) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= int(s)
    nbytes = n * torch.empty(0, dtype=dtype).element_size()
    raw = torch.as_tensor(_DevMem(ptr, max(nbytes, 1), owner), device=device)
    return raw[:nbytes].view(dtype).view(*shape)


def pull_rows(dst: torch.Tensor, src_ptr: int, src_pitch_bytes: int) -> None:
    """Copy ``dst.shape[0]`` row segments of ``dst.shape[1]`` elements from (peer) memory at ``src_ptr``
    (segment r starts ``r * src_pitch_bytes`` further) into the 2-D view ``dst`` (unit inner stride),
    with this library's own copy kernel on the current stream: a remote tile that several CTAs are
    going to read crosses NVLink once."""
    assert dst.dim() == 2 and dst.stride(1) == 1 and dst.is_cuda
    es = dst.element_size()
    rc = nv.lib("peer_rt").omni_peer_copy_2d(
        ctypes.c_void_p(dst.data_ptr()), ctypes.c_size_t(dst.stride(0) * es), ctypes.c_void_p(src_ptr),
        ctypes.c_size_t(src_pitch_bytes), ctypes.c_size_t(dst.shape[1] * es), ctypes.c_long(dst.shape[0]), nv.stream_ptr())
    nv.check_rc(rc, "omni_peer_copy_2d")


class SymTensor:
    """A symmetric allocation: the local tensor and the device pointer of its twin on every rank."""

    def __init__(self, local: torch.Tensor, ptrs: list[int], offset: int):
        self.local = local
        self.ptrs = ptrs          # index = rank in group; ptrs[my_rank] == local.data_ptr()
        self.offset = offset

    def peer_ptrs(self, byte_offset: int = 0) -> list[int]:
        return [p + byte_offset for p in self.ptrs]


class OmniSync(ctypes.Structure):
    """C mirror of ``OmniSync`` in csrc/peer_signal.cuh: what a launch reports to the group after its
    peer stores (``signal_*``) and what it waits for before reading peer-written data (``wait_*``)."""
    _fields_ = [("signal_counters", ctypes.c_void_p * 16), ("signal_done", ctypes.c_void_p),
                ("signal_n", ctypes.c_int), ("wait_counter", ctypes.c_void_p), ("wait_epoch", ctypes.c_void_p),
                ("wait_per_use", ctypes.c_ulonglong), ("wait_timeout_ns", ctypes.c_ulonglong)]


class SignalChannel:
    """One direction of a fused exchange: producers on every rank report an arrival per launch,
    the consumer kernel on every rank waits for ``per_use`` arrivals (producer launches x ranks).

    ``counter`` lives in the arena (peers add to it); ``done`` (producer CTA count) and ``epoch``
    (consumer uses completed, CTA exit count) are local device words, so a captured CUDA graph
    replays correctly: nothing in the launch arguments changes from use to use."""

    def __init__(self, arena: "PeerArena | None", producer_launches: int = 1, device=None, timeout_ms: int = 1000):
        """``arena=None``: a single-rank channel on ``device`` (one GPU; used by tests and by groups of
        one), whose counter is an ordinary device tensor."""
        self.arena = arena
        if arena is not None:
            self.counter = arena.alloc((16,), torch.int64)      # [0] is the arrival counter; the rest pads a line
            world, device, timeout_ns = arena.world, arena.device, arena.timeout_ns
        else:
            t = torch.zeros(16, dtype=torch.int64, device=device)
            self.counter = SymTensor(t, [t.data_ptr()], 0)
            world, timeout_ns = 1, int(timeout_ms) * 1_000_000
        self.counter.local.zero_()
        self.done = torch.zeros(4, dtype=torch.int32, device=device)
        self.epoch = torch.zeros(2, dtype=torch.int64, device=device)
        self.per_use = producer_launches * world
        self._signal = OmniSync()
        for r, p in enumerate(self.counter.ptrs):
            self._signal.signal_counters[r] = p
        self._signal.signal_done = self.done.data_ptr()
        self._signal.signal_n = world
        self._wait = OmniSync()
        self._wait.wait_counter = self.counter.local.data_ptr()
        self._wait.wait_epoch = self.epoch.data_ptr()
        self._wait.wait_per_use = self.per_use
        self._wait.wait_timeout_ns = timeout_ns

    def signal(self) -> OmniSync:
        """For the producer launch (reports one arrival to every rank when its stores are out)."""
        return self._signal

    def wait(self) -> OmniSync:
        """For the consumer launch (waits for this use's arrivals before reading)."""
        return self._wait

    @staticmethod
    def combine(wait_from: "SignalChannel | None", signal_to: "SignalChannel | None") -> OmniSync | None:
        """A launch that consumes one exchange and produces the next."""
        if wait_from is None and signal_to is None:
            return None
        s = OmniSync()
        if signal_to is not None:
            ctypes.memmove(ctypes.byref(s), ctypes.byref(signal_to._signal), ctypes.sizeof(OmniSync))
        if wait_from is not None:
            s.wait_counter, s.wait_epoch = wait_from._wait.wait_counter, wait_from._wait.wait_epoch
            s.wait_per_use, s.wait_timeout_ns = wait_from._wait.wait_per_use, wait_from._wait.wait_timeout_ns
        return s


class PeerArena:
    def __init__(self, group, nbytes: int, device: torch.device | None = None, timeout_ms: int = 1000):
        """``group``: a GroupCoordinator (uses its CPU twin to exchange IPC handles)."""
        self.group = group
        self.rank, self.world = group.rank_in_group, group.world_size
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        # OMNI_PEER_CANARY=1 (debug / tests): a guard block filled with a pattern follows every
        # allocation and is verified on the host by check_canaries() / close(), so a kernel that
        # stores past the end of a peer buffer is caught without any device-side trap
        self._canary = os.environ.get("OMNI_PEER_CANARY") == "1"
        self._guards: list[int] = []
        self.nbytes = (int(nbytes) + _ALIGN - 1) // _ALIGN * _ALIGN + (64 * _ALIGN if self._canary else 0)
        self.timeout_ns = int(timeout_ms) * 1_000_000
        self._lib = nv.lib("peer_rt")
        self._flag_bytes = _ALIGN                      # world u64 flags + the epoch counter
        total = self.nbytes + self._flag_bytes
        base = ctypes.c_void_p()
        nv.check_rc(self._lib.omni_peer_alloc(ctypes.c_size_t(total), ctypes.byref(base)), "omni_peer_alloc")
        self._base = base.value
        hsz = self._lib.omni_ipc_handle_size()
        handle = (ctypes.c_ubyte * hsz)()
        nv.check_rc(self._lib.omni_peer_export(ctypes.c_void_p(self._base), handle), "omni_peer_export")
        handles = group.all_gather_object(bytes(handle))
        self.bases: list[int] = []
        self._opened: list[int] = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.bases.append(self._base)
                continue
            buf = (ctypes.c_ubyte * hsz).from_buffer_copy(h)
            p = ctypes.c_void_p()
            nv.check_rc(self._lib.omni_peer_open(buf, ctypes.byref(p)), "omni_peer_open")
            self.bases.append(p.value)
            self._opened.append(p.value)
        # flag page sits at the start of every arena; the epoch counter after the flags
        self._flag_ptrs = (ctypes.c_void_p * self.world)(*self.bases)
        self._epoch_ptr = self._base + 8 * 16
        self._bump = self._flag_bytes
        self._closed = False
        group.barrier()

    def alloc(self, shape, dtype=torch.bfloat16) -> SymTensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        off = self._bump
        if off + nbytes > self.nbytes + self._flag_bytes:
            raise MemoryError(f"peer arena exhausted: need {nbytes} B at offset {off}, arena {self.nbytes} B")
        self._bump = (off + nbytes + _ALIGN - 1) // _ALIGN * _ALIGN
        if self._canary and self._bump + _ALIGN <= self.nbytes + self._flag_bytes:
            g = self._bump
            tensor_from_ptr(self._base + g, (_ALIGN,), torch.uint8, self.device, owner=self).fill_(_CANARY_BYTE)
            self._guards.append(g)
            self._bump += _ALIGN
        local = tensor_from_ptr(self._base + off, shape, dtype, self.device, owner=self)
        return SymTensor(local, [b + off for b in self.bases], off)

    def check_canaries(self) -> list[int]:
        """Offsets of guard blocks (this rank's arena) that no longer hold the pattern."""
        bad = []
        for g in self._guards:
            t = tensor_from_ptr(self._base + g, (_ALIGN,), torch.uint8, self.device, owner=self)
            if not bool((t == _CANARY_BYTE).all().item()):
                bad.append(g)
        return bad

    def barrier(self) -> None:
        """Device-side barrier over the group on the current stream (bounded wait)."""
        if self.world == 1:
            return
        st = nv.status_word(self.device)
        rc = self._lib.omni_peer_barrier(self._flag_ptrs, ctypes.c_int(self.rank), ctypes.c_int(self.world),
                                         ctypes.c_void_p(self._epoch_ptr), ctypes.c_ulonglong(self.timeout_ns),
                                         nv.ptr(st), nv.stream_ptr())
        nv.check_rc(rc, "omni_peer_barrier")

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        torch.cuda.synchronize(self.device)
        try:
            self.group.barrier()
        except Exception:
            pass
        bad = self.check_canaries() if self._canary else []
        for p in self._opened:
            self._lib.omni_peer_close(ctypes.c_void_p(p))
        self._lib.omni_peer_free(ctypes.c_void_p(self._base))
        if bad:
            raise RuntimeError(f"peer arena guard blocks overwritten at offsets {bad} (rank {self.rank})")
