"""In-process connector: stages that live in one process hand objects over by reference
(GPU tensors stay on the GPU).  Also the fake used by the connector unit tests, in the
spirit of the reference's MockConnector (tests/distributed/omni_connectors/test_kv_flow.py:14-29)."""
from __future__ import annotations

import threading
import time

from .base import OmniConnectorBase


class InProcConnector(OmniConnectorBase):
    supports_device_tensors = True

    def __init__(self, config=None):
        super().__init__(config)
        self._store: dict[str, object] = {}
        self._cv = threading.Condition()
        self.get_timeout = float(self.config.get("get_timeout_s", 3.0))

    @staticmethod
    def _nbytes(o) -> int:
        import torch
        if isinstance(o, torch.Tensor):
            return o.numel() * o.element_size()
        if isinstance(o, dict):
            return sum(InProcConnector._nbytes(v) for v in o.values())
        if isinstance(o, (list, tuple)):
            return sum(InProcConnector._nbytes(v) for v in o)
        return 0

    def put(self, from_stage, to_stage, key, data):
        k = self.make_key(from_stage, to_stage, key)
        with self._cv:
            self._store[k] = data
            self._cv.notify_all()
        n = self._nbytes(data)
        self.stats["puts"] += 1
        self.stats["bytes"] += n
        return True, n, {"inproc_key": k}

    def get(self, from_stage, to_stage, key, metadata=None):
        k = self.make_key(from_stage, to_stage, key)
        deadline = time.monotonic() + self.get_timeout
        with self._cv:
            while k not in self._store:
                rem = deadline - time.monotonic()
                if rem <= 0:
                    return None
                self._cv.wait(rem)
            data = self._store.pop(k)
        self.stats["gets"] += 1
        return data, self._nbytes(data)

    def cleanup(self, key):
        with self._cv:
            for k in [k for k in self._store if k.endswith(key)]:
                self._store.pop(k, None)

    def cleanup_all(self):
        with self._cv:
            self._store.clear()
