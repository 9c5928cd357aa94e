"""Device-to-device connector (K13): payload tensors stay in GPU memory.

Same process: tensors are handed over by reference.  Across processes on one NVSwitch box: the
producer copies tensors into a peer-mapped staging arena of the CONSUMER (csrc/peer_rt.cu IPC
mapping; the copy is a plain device kernel / cudaMemcpyAsync over NVLink) and only a small
descriptor {offset, shape, dtype} travels through the control queue.  The reference moves
every hand-off GPU -> CPU -> msgpack -> shm -> CPU -> GPU
(vllm_omni/worker/gpu_ar_model_runner.py:525-568, serialization.py).
"""
from __future__ import annotations

import threading
import time

import torch

from .base import OmniConnectorBase

_DT = {torch.bfloat16: "bf16", torch.float16: "f16", torch.float32: "f32", torch.int64: "i64", torch.int32: "i32",
       torch.uint8: "u8", torch.bool: "b"}
_TD = {v: k for k, v in _DT.items()}


class DeviceConnector(OmniConnectorBase):
    supports_device_tensors = True

    def __init__(self, config=None):
        super().__init__(config)
        self._store: dict[str, object] = {}
        self._cv = threading.Condition()
        self.get_timeout = float(self.config.get("get_timeout_s", 3.0))
        self.arena = None                    # PeerArena when the two stages are different processes
        self._bump = 0

    def attach_arena(self, arena) -> None:
        """``arena``: a PeerArena over the (producer, consumer) pair; index 1 is the consumer."""
        self.arena = arena

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
