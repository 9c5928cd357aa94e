"""Fault injection at the connector seam (host side only): a wrapper around any connector that
drops, delays, loses or corrupts payloads on a schedule, for exercising the error paths of the
orchestrator, the KV-transfer manager and the chunk adapter without touching a GPU.

    runtime:
      connectors:
        flaky:
          name: FaultInjectionConnector
          extra:
            inner: {name: SharedMemoryConnector, extra: {get_retries: 2, get_retry_interval_s: 0.01}}
            schedule: [null, drop_put, corrupt, lose_get]     # one entry per call, then ``rates`` apply
            rates: {drop_put: 0.0, lose_get: 0.0, corrupt: 0.0}
            delay_ms: 5
            seed: 0

``drop_put``: the put reports failure (nothing stored).  ``corrupt``: one byte of the stored payload
is flipped after the put, so the receiver's checksum test fires.  ``lose_get``: the payload is
removed before the get, which then runs out of retries and returns None (the adapter raises
``TimeoutError``).  ``delay_ms`` sleeps before every put and get.

The reference has no fault-injection hooks (its reliability tests are only planned); its bounded
connector retries and KV-transfer timeouts are the behaviour these faults drive.
"""
from __future__ import annotations

import random
import time
from multiprocessing import shared_memory

from .base import OmniConnectorBase


class FaultInjectingConnector(OmniConnectorBase):
    FAULTS = ("drop_put", "corrupt", "lose_get")

    def __init__(self, config: dict | None = None, inner: OmniConnectorBase | None = None):
        super().__init__(config)
        if inner is None:
            from .factory import OmniConnectorFactory
            inner = OmniConnectorFactory.create(self.config.get("inner") or "InProcConnector")
        self.inner = inner
        self.supports_device_tensors = inner.supports_device_tensors
        self.schedule = list(self.config.get("schedule") or [])
        self.rates = {k: float(v) for k, v in (self.config.get("rates") or {}).items()}
        self.delay_s = float(self.config.get("delay_ms", 0.0)) / 1e3
        self.rng = random.Random(int(self.config.get("seed", 0)))
        self.injected: list[tuple[str, str]] = []          # (fault, key) log for assertions

    def _next(self, allowed):
        if self.schedule:
            f = self.schedule.pop(0)
            return f if f in allowed else None
        for f in allowed:
            if self.rates.get(f, 0.0) > 0 and self.rng.random() < self.rates[f]:
                return f
        return None

    def put(self, from_stage, to_stage, key, data):
        if self.delay_s:
            time.sleep(self.delay_s)
        fault = self._next(("drop_put", "corrupt"))
        if fault == "drop_put":
            self.injected.append((fault, key))
            self.stats["errors"] += 1
            return False, 0, None
        ok, size, meta = self.inner.put(from_stage, to_stage, key, data)
        if ok and fault == "corrupt" and self._corrupt(meta):
            self.injected.append((fault, key))
        self.stats["puts"] += int(ok)
        return ok, size, meta

    def _corrupt(self, meta) -> bool:
        if not meta:
            return False
        if "inline_bytes" in meta and meta["inline_bytes"]:
            b = bytearray(meta["inline_bytes"])
            b[len(b) // 2] ^= 0x5A
            meta["inline_bytes"] = bytes(b)
            return True
        if "shm" in meta:
            try:
                shm = shared_memory.SharedMemory(name=meta["shm"]["name"])
                shm.buf[meta["shm"]["size"] // 2] ^= 0x5A
                shm.close()
                return True
            except FileNotFoundError:
                return False
        return False

    def get(self, from_stage, to_stage, key, metadata=None):
        if self.delay_s:
            time.sleep(self.delay_s)
        if self._next(("lose_get",)) == "lose_get":
            self.injected.append(("lose_get", key))
            self.inner.cleanup(key)
            md = dict(metadata or {})
            md.pop("inline_bytes", None)
            if "shm" in md:                                  # the segment is gone; the name no longer resolves
                md["shm"] = {"name": md["shm"]["name"] + "_lost", "size": md["shm"]["size"]}
            out = self.inner.get(from_stage, to_stage, key, md)
            if out is None:
                self.stats["errors"] += 1
            return out
        out = self.inner.get(from_stage, to_stage, key, metadata)
        self.stats["gets"] += int(out is not None)
        return out

    def cleanup(self, key):
        self.inner.cleanup(key)

    def cleanup_all(self):
        self.inner.cleanup_all()

    def health(self):
        h = self.inner.health()
        h["injected_faults"] = len(self.injected)
        return h
