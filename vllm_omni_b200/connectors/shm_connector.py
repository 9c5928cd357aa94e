"""POSIX shared-memory connector (vllm_omni/.../connectors/shm_connector.py): payloads at or
above ``shm_threshold_bytes`` go into a named segment and only {name, size} travels through
the control queue; smaller ones ride inline.  ``get`` retries (30 x 100 ms by default) so
a consumer can race the producer; a CRC guards against torn or corrupted segments.
"""
from __future__ import annotations

import time
import zlib
from multiprocessing import shared_memory
from typing import Any

from .base import OmniConnectorBase
from .serialization import OmniSerializer


class SharedMemoryConnector(OmniConnectorBase):
    def __init__(self, config: dict | None = None):
        super().__init__(config)
        self.threshold = int(self.config.get("shm_threshold_bytes", 65536))
        self.retries = int(self.config.get("get_retries", 30))
        self.retry_interval = float(self.config.get("get_retry_interval_s", 0.1))
        self._owned: dict[str, str] = {}        # key -> segment name
        self._inline: dict[str, bytes] = {}

    def put(self, from_stage, to_stage, key, data):
        try:
            blob = OmniSerializer.serialize(data)
            k = self.make_key(from_stage, to_stage, key)
            size = len(blob)
            meta = {"size": size, "crc": zlib.crc32(blob) & 0xFFFFFFFF}
            if size >= self.threshold:
                shm = shared_memory.SharedMemory(create=True, size=max(size, 1))
                shm.buf[:size] = blob
                meta["shm"] = {"name": shm.name, "size": size}
                self._owned[k] = shm.name
                shm.close()
            else:
                meta["inline_bytes"] = blob
                self._inline[k] = blob
            self.stats["puts"] += 1
            self.stats["bytes"] += size
            return True, size, meta
        except Exception:
            self.stats["errors"] += 1
            return False, 0, None

    def get(self, from_stage, to_stage, key, metadata: dict | None = None):
        k = self.make_key(from_stage, to_stage, key)
        for attempt in range(max(1, self.retries)):
            blob = None
            if metadata and "inline_bytes" in metadata:
                blob = metadata["inline_bytes"]
            elif metadata and "shm" in metadata:
                try:
                    shm = shared_memory.SharedMemory(name=metadata["shm"]["name"])
                    blob = bytes(shm.buf[:metadata["shm"]["size"]])
                    shm.close()
                    try:
                        shm.unlink()
                    except FileNotFoundError:
                        pass
                    self._owned.pop(k, None)
                except FileNotFoundError:
                    blob = None
            elif k in self._inline:
                blob = self._inline.pop(k)
            if blob is not None:
                if metadata and "crc" in metadata and (zlib.crc32(blob) & 0xFFFFFFFF) != metadata["crc"]:
                    self.stats["errors"] += 1
                    raise ValueError(f"connector payload {k} failed its checksum")
                self.stats["gets"] += 1
                return OmniSerializer.deserialize(blob), len(blob)
            if attempt + 1 < self.retries:
                time.sleep(self.retry_interval)
        return None

    def cleanup(self, key: str) -> None:
        for k in [k for k in self._owned if k.endswith(key)]:
            self._unlink(self._owned.pop(k))
        for k in [k for k in self._inline if k.endswith(key)]:
            self._inline.pop(k, None)

    def cleanup_all(self) -> None:
        for name in list(self._owned.values()):
            self._unlink(name)
        self._owned.clear()
        self._inline.clear()

    @staticmethod
    def _unlink(name: str):
        try:
            shm = shared_memory.SharedMemory(name=name)
            shm.close()
            shm.unlink()
        except FileNotFoundError:
            pass
