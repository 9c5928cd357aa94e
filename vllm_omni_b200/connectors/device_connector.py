"""Device-to-device connector (K13): payload tensors stay in GPU memory.

Same process: tensors are handed over by reference.

Across processes on one NVSwitch box (``cross_process: true``): the CONSUMER stage owns a receive
arena in its GPU's memory (``cudaMalloc``, exported as a CUDA IPC handle).  The handle and the
arena's allocation ring live in a small POSIX shared-memory control block named after the edge
(``<name>_<from>_<to>``), which is how the two processes find each other.  ``put`` (producer)
maps the consumer's arena once, reserves a range in the ring, PUSHES every tensor of the payload
into it with a copy kernel of this library (csrc/peer_rt.cu ``omni_peer_copy``: plain 16-byte peer
stores over NVLink, no library copy is handed the peer pointer), waits for the copies, and returns
a descriptor {entry, offsets, shapes, dtypes, tree}; the descriptor is what travels through the
stage control plane.  ``get`` (consumer) rebuilds the payload from its OWN arena with local copies
and frees the range.  One producer and one consumer per edge.

The reference moves every hand-off GPU -> CPU -> msgpack -> shm -> CPU -> GPU
(vllm_omni/worker/gpu_ar_model_runner.py:525-568, serialization.py,
omni_connectors/kv_transfer_manager.py:217-276).
"""
from __future__ import annotations

import ctypes
import struct
import threading
import time
from multiprocessing import shared_memory

import torch

from .base import OmniConnectorBase

_DT = {torch.bfloat16: "bf16", torch.float16: "f16", torch.float32: "f32", torch.int64: "i64", torch.int32: "i32",
       torch.uint8: "u8", torch.bool: "b"}
_TD = {v: k for k, v in _DT.items()}


class ArenaRing:
    """Allocation ring over the consumer's arena, kept in a shared-memory control block so that the
    producer (reserves ranges) and the consumer (frees them, in any order) see the same state.

    Layout (little endian): magic u64 | arena_bytes u64 | ready u64 | ipc handle 64 B | head_entry
    u64 | tail_entry u64 | head_off u64 | entries[N] of (offset u64, size u64, state u64).  Entries
    are handed out in order by the producer (state 1 = in use); the consumer sets state 2 = free;
    the producer retires leading free entries to get their bytes back.  One writer per field."""
    MAGIC, N, HDR = 0x4F4D4E4944435631, 1024, 8 * 3 + 64 + 8 * 3
    ALIGN = 256

    def __init__(self, name: str, create: bool, arena_bytes: int = 0, handle: bytes = b""):
        size = self.HDR + self.N * 24
        self.name = name
        if create:
            try:
                self.shm = shared_memory.SharedMemory(name=name, create=True, size=size)
            except FileExistsError:                      # a stale block of an earlier run
                old = shared_memory.SharedMemory(name=name)
                old.close()
                old.unlink()
                self.shm = shared_memory.SharedMemory(name=name, create=True, size=size)
            self.shm.buf[:size] = bytes(size)
            struct.pack_into("<QQ", self.shm.buf, 0, self.MAGIC, arena_bytes)
            self.shm.buf[24:24 + 64] = handle.ljust(64, b"\0")[:64]
            struct.pack_into("<Q", self.shm.buf, 16, 1)          # ready
        else:
            self.shm = shared_memory.SharedMemory(name=name)
        self.owner = create

    # field access ------------------------------------------------------------
    def _g(self, off):
        return struct.unpack_from("<Q", self.shm.buf, off)[0]

    def _s(self, off, v):
        struct.pack_into("<Q", self.shm.buf, off, v)

    @property
    def ready(self):
        return self._g(0) == self.MAGIC and self._g(16) == 1

    @property
    def arena_bytes(self):
        return self._g(8)

    @property
    def handle(self) -> bytes:
        return bytes(self.shm.buf[24:24 + 64])

    def _entry(self, i):
        return struct.unpack_from("<QQQ", self.shm.buf, self.HDR + (i % self.N) * 24)

    def _set_entry(self, i, off, size, state):
        struct.pack_into("<QQQ", self.shm.buf, self.HDR + (i % self.N) * 24, off, size, state)

    # producer ----------------------------------------------------------------
    def reserve(self, nbytes: int) -> tuple[int, int] | None:
        """Returns (entry index, byte offset) of a range of ``nbytes``, or None when the arena (or
        the entry table) is full right now."""
        nbytes = (nbytes + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        cap = self.arena_bytes
        if nbytes > cap:
            raise ValueError(f"payload of {nbytes} B exceeds the connector arena ({cap} B); raise arena_mb")
        H, T, O = self.HDR - 24, self.HDR - 16, self.HDR - 8
        head, tail = self._g(H), self._g(T)
        while tail < head and self._entry(tail)[2] == 2:          # retire ranges the consumer has freed
            tail += 1
        self._s(T, tail)
        if head - tail >= self.N:
            return None
        if tail == head:                                          # empty: start over at the front
            off, ok = 0, True
        else:
            lo = self._entry(tail)[0]                             # oldest live byte
            last_off, last_size, _ = self._entry(head - 1)
            off = last_off + last_size                            # end of the newest range
            if last_off >= lo:                                    # live data does not wrap: [lo, off)
                if off + nbytes <= cap:
                    ok = True
                elif nbytes <= lo:                                # wrap to the front
                    off, ok = 0, True
                else:
                    ok = False
            else:                                                 # live data wraps: the free gap is [off, lo)
                ok = off + nbytes <= lo
        if not ok:
            return None
        self._set_entry(head, off, nbytes, 1)
        self._s(O, off + nbytes)
        self._s(H, head + 1)
        return head, off

    # consumer ----------------------------------------------------------------
    def release(self, entry: int) -> None:
        off, size, _ = self._entry(entry)
        self._set_entry(entry, off, size, 2)

    def close(self):
        try:
            self.shm.close()
            if self.owner:
                self.shm.unlink()
        except Exception:   # noqa: BLE001
            pass


class DeviceConnector(OmniConnectorBase):
    supports_device_tensors = True

    def __init__(self, config=None):
        super().__init__(config)
        self._store: dict[str, object] = {}
        self._cv = threading.Condition()
        self.get_timeout = float(self.config.get("get_timeout_s", 3.0))
        self.cross_process = bool(self.config.get("cross_process", False))
        self.arena_bytes = int(float(self.config.get("arena_mb", 256)) * (1 << 20))
        self.name = str(self.config.get("name", "omni_dc"))
        self._rx: dict[str, tuple] = {}          # consumer side: edge -> (ring, arena base ptr, arena tensor)
        self._tx: dict[str, tuple] = {}          # producer side: edge -> (ring, mapped peer base ptr)

    # ------------------------------------------------------------------ cross-process plumbing
    def _edge(self, from_stage, to_stage) -> str:
        return f"{self.name}_{from_stage}_{to_stage}"

    def open_receiver(self, from_stage, to_stage, device=None) -> None:
        """Consumer side: allocate and publish the receive arena of this edge (idempotent).  Called
        by the consumer stage at start-up, or lazily by the first ``get``."""
        edge = self._edge(from_stage, to_stage)
        if edge in self._rx:
            return
        from ..ops import _native as nv
        lib = nv.lib("peer_rt")
        dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        with torch.cuda.device(dev):
            base = ctypes.c_void_p()
            nv.check_rc(lib.omni_peer_alloc(ctypes.c_size_t(self.arena_bytes), ctypes.byref(base)), "omni_peer_alloc")
            hsz = lib.omni_ipc_handle_size()
            handle = (ctypes.c_ubyte * hsz)()
            nv.check_rc(lib.omni_peer_export(base, handle), "omni_peer_export")
        from ..parallel.peer_memory import tensor_from_ptr
        view = tensor_from_ptr(base.value, (self.arena_bytes,), torch.uint8, dev, owner=self)
        ring = ArenaRing(edge, create=True, arena_bytes=self.arena_bytes, handle=bytes(handle))
        self._rx[edge] = (ring, base.value, view, dev)

    def _sender(self, from_stage, to_stage):
        edge = self._edge(from_stage, to_stage)
        tx = self._tx.get(edge)
        if tx is not None:
            return tx
        deadline = time.monotonic() + float(self.config.get("connect_timeout_s", 30.0))
        ring = None
        while ring is None:
            try:
                r = ArenaRing(edge, create=False)
                if r.ready:
                    ring = r
                else:
                    r.close()
            except FileNotFoundError:
                pass
            if ring is None:
                if time.monotonic() > deadline:
                    raise TimeoutError(f"device connector: the consumer of edge {edge!r} never published its arena")
                time.sleep(0.01)
        from ..ops import _native as nv
        lib = nv.lib("peer_rt")
        hsz = lib.omni_ipc_handle_size()
        buf = (ctypes.c_ubyte * hsz).from_buffer_copy(ring.handle[:hsz])
        p = ctypes.c_void_p()
        nv.check_rc(lib.omni_peer_open(buf, ctypes.byref(p)), "omni_peer_open")
        tx = self._tx[edge] = (ring, p.value)
        return tx

    def _put_cross(self, from_stage, to_stage, key, data):
        from ..ops import _native as nv
        ring, peer_base = self._sender(from_stage, to_stage)
        tensors: list[torch.Tensor] = []

        def note(t):
            tensors.append(t.detach().contiguous())
            return {"__t__": len(tensors) - 1}
        tree = self._walk(data, note)
        A = ArenaRing.ALIGN
        offs, total = [], 0
        for t in tensors:
            offs.append(total)
            total += (t.numel() * t.element_size() + A - 1) // A * A
        deadline = time.monotonic() + self.get_timeout
        got = ring.reserve(max(total, A))
        while got is None:
            if time.monotonic() > deadline:
                self.stats["errors"] += 1
                return False, 0, {"error": "device connector arena full"}
            time.sleep(0.0005)
            got = ring.reserve(max(total, A))
        entry, base_off = got
        lib = nv.lib("peer_rt")
        for t, o in zip(tensors, offs):      # host tensors (small: lengths, ids) ride in the descriptor instead
            n = t.numel() * t.element_size()
            if t.is_cuda and n:
                with torch.cuda.device(t.device):
                    nv.check_rc(lib.omni_peer_copy(ctypes.c_void_p(peer_base + base_off + o), nv.ptr(t),
                                                   ctypes.c_size_t(n), nv.stream_ptr()), "omni_peer_copy")
        devs = {t.device for t in tensors if t.is_cuda}
        for d in devs:
            torch.cuda.current_stream(d).synchronize()          # the descriptor must not overtake the data
        desc = {"entry": entry, "offset": base_off, "tree": tree,
                "tensors": [{"off": o, "shape": list(t.shape), "dtype": _DT[t.dtype],
                             "host": None if t.is_cuda else t.tolist()} for t, o in zip(tensors, offs)]}
        self.stats["puts"] += 1
        self.stats["bytes"] += total
        return True, total, {"device_desc": desc}

    def _get_cross(self, from_stage, to_stage, key, metadata):
        desc = (metadata or {}).get("device_desc")
        if desc is None:
            return None
        self.open_receiver(from_stage, to_stage)
        ring, _base, view, dev = self._rx[self._edge(from_stage, to_stage)]
        outs = []
        n = 0
        for td in desc["tensors"]:
            dt = _TD[td["dtype"]]
            if td["host"] is not None:
                outs.append(torch.tensor(td["host"], dtype=dt).reshape(td["shape"]))
                continue
            cnt = 1
            for s_ in td["shape"]:
                cnt *= int(s_)
            nb = cnt * torch.empty(0, dtype=dt).element_size()
            a = desc["offset"] + td["off"]
            outs.append(view[a:a + nb].view(dt).view(td["shape"]).clone())      # local copy out of the arena
            n += nb
        torch.cuda.current_stream(dev).synchronize()
        ring.release(desc["entry"])
        payload = self._unwalk(desc["tree"], outs)
        self.stats["gets"] += 1
        return payload, n

    @staticmethod
    def _unwalk(o, tensors):
        if isinstance(o, dict):
            if set(o) == {"__t__"}:
                return tensors[o["__t__"]]
            return {k: DeviceConnector._unwalk(v, tensors) for k, v in o.items()}
        if isinstance(o, (list, tuple)):
            return type(o)(DeviceConnector._unwalk(v, tensors) for v in o)
        return o

    @staticmethod
    def _walk(o, fn):
        if isinstance(o, torch.Tensor):
            return fn(o)
        if isinstance(o, dict):
            return {k: DeviceConnector._walk(v, fn) for k, v in o.items()}
        if isinstance(o, (list, tuple)):
            return type(o)(DeviceConnector._walk(v, fn) for v in o)
        return o

    def put(self, from_stage, to_stage, key, data):
        if self.cross_process:
            return self._put_cross(from_stage, to_stage, key, data)
        k = self.make_key(from_stage, to_stage, key)
        nbytes = [0]

        def keep(t):
            nbytes[0] += t.numel() * t.element_size()
            return t.detach()
        payload = self._walk(data, keep)
        if torch.cuda.is_available():
            ev = torch.cuda.Event()
            ev.record()
        else:
            ev = None
        with self._cv:
            self._store[k] = (payload, ev)
            self._cv.notify_all()
        self.stats["puts"] += 1
        self.stats["bytes"] += nbytes[0]
        return True, nbytes[0], {"device_key": k}

    def get(self, from_stage, to_stage, key, metadata=None):
        if self.cross_process:
            return self._get_cross(from_stage, to_stage, key, metadata)
        k = self.make_key(from_stage, to_stage, key)
        deadline = time.monotonic() + self.get_timeout
        with self._cv:
            while k not in self._store:
                rem = deadline - time.monotonic()
                if rem <= 0:
                    return None
                self._cv.wait(rem)
            payload, ev = self._store.pop(k)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)      # order the consumer after the producer's writes
        n = [0]
        self._walk(payload, lambda t: n.__setitem__(0, n[0] + t.numel() * t.element_size()) or t)
        self.stats["gets"] += 1
        return payload, n[0]

    def cleanup(self, key):
        with self._cv:
            for k in [k for k in self._store if k.endswith(key)]:
                self._store.pop(k, None)

    def cleanup_all(self):
        with self._cv:
            self._store.clear()

    def close(self) -> None:
        self.cleanup_all()
        if self._tx or self._rx:
            from ..ops import _native as nv
            lib = nv.lib("peer_rt")
            for ring, p in self._tx.values():
                lib.omni_peer_close(ctypes.c_void_p(p))
                ring.close()
            for ring, base, _view, dev in self._rx.values():
                torch.cuda.synchronize(dev)
                lib.omni_peer_free(ctypes.c_void_p(base))
                ring.close()
            self._tx, self._rx = {}, {}
