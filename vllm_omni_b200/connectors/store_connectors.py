"""Connectors backed by external stores (vllm_omni/.../connectors/mooncake_connector.py,
yuanrong_connector.py).  Neither client library is installed in this image; the classes keep
the configuration surface and fail with a clear message when constructed without the library,
so stage configs that name them are diagnosed at start-up instead of at the first transfer."""
from __future__ import annotations

import time

from .base import OmniConnectorBase
from .serialization import OmniSerializer


class _StoreConnector(OmniConnectorBase):
    LIB = ""
    RETRIES, INTERVAL = 20, 0.05

    def __init__(self, config=None, client=None):
        super().__init__(config)
        self.client = client if client is not None else self._make_client()

    def _make_client(self):
        raise NotImplementedError

    def put(self, from_stage, to_stage, key, data):
        try:
            blob = OmniSerializer.serialize(data)
            self.client.put(self.make_key(from_stage, to_stage, key), blob)
            self.stats["puts"] += 1
            self.stats["bytes"] += len(blob)
            return True, len(blob), {"store_key": self.make_key(from_stage, to_stage, key)}
        except Exception:
            self.stats["errors"] += 1
            return False, 0, None

    def get(self, from_stage, to_stage, key, metadata=None):
        k = self.make_key(from_stage, to_stage, key)
        for _ in range(self.RETRIES):
            blob = self.client.get(k)
            if blob:
                self.stats["gets"] += 1
                return OmniSerializer.deserialize(bytes(blob)), len(blob)
            time.sleep(self.INTERVAL)
        return None

    def cleanup(self, key):
        try:
            self.client.remove(key)
        except Exception:
            pass


class MooncakeConnector(_StoreConnector):
    LIB = "mooncake"

    def _make_client(self):
        try:
            from mooncake.store import MooncakeDistributedStore     # type: ignore
        except ImportError as e:
            raise RuntimeError("MooncakeConnector needs the `mooncake` package, which is not installed; use "
                               "SharedMemoryConnector or DeviceConnector on a single node") from e
        c = MooncakeDistributedStore()
        cfg = self.config
        c.setup(cfg.get("host", "127.0.0.1"), cfg.get("metadata_server", ""), cfg.get("segment", 512 << 20),
                cfg.get("localbuf", 64 << 20), cfg.get("protocol", "tcp"), cfg.get("device_name", ""),
                cfg.get("master", "127.0.0.1:50051"))
        return c


class YuanrongConnector(_StoreConnector):
    LIB = "datasystem"

    def _make_client(self):
        try:
            from datasystem import DsClient     # type: ignore
        except ImportError as e:
            raise RuntimeError("YuanrongConnector needs the `datasystem` package, which is not installed; use "
                               "SharedMemoryConnector or DeviceConnector on a single node") from e
        c = DsClient(self.config.get("host", "127.0.0.1"), int(self.config.get("port", 31501)))
        c.init()
        return c
