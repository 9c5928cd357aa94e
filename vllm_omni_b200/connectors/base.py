"""OmniConnector interface: a keyed put/get store between stages
(vllm_omni/distributed/omni_connectors/connectors/base.py).

``put(from_stage, to_stage, key, data) -> (ok, size_bytes, metadata)`` and
``get(from_stage, to_stage, key, metadata) -> (data, size_bytes) | None``.  Host connectors
serialise; the device connector (``device_connector.py``) moves tensors GPU-to-GPU and only
sends a small descriptor through the control plane.
"""
from __future__ import annotations

import abc
from typing import Any


class OmniConnectorBase(abc.ABC):
    supports_device_tensors = False

    def __init__(self, config: dict | None = None):
        self.config = dict(config or {})
        self.stats = {"puts": 0, "gets": 0, "bytes": 0, "errors": 0}

    @staticmethod
    def make_key(from_stage, to_stage, key: str) -> str:
        return f"{from_stage}_{to_stage}_{key}"

    @abc.abstractmethod
    def put(self, from_stage, to_stage, key: str, data: Any) -> tuple[bool, int, dict | None]:
        ...

    @abc.abstractmethod
    def get(self, from_stage, to_stage, key: str, metadata: dict | None = None):
        ...

    def cleanup(self, key: str) -> None:
        pass

    def cleanup_all(self) -> None:
        pass

    def health(self) -> dict:
        return {"status": "ok", **self.stats}

    def close(self) -> None:
        self.cleanup_all()
