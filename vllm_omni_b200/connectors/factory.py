"""Connector registry and per-edge construction
(vllm_omni/distributed/omni_connectors/factory.py, utils/initialization.py, utils/config.py)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

from .base import OmniConnectorBase


@dataclass
class ConnectorSpec:
    name: str = "SharedMemoryConnector"
    extra: dict[str, Any] = field(default_factory=dict)


class OmniConnectorFactory:
    _registry: dict[str, Callable[[dict], OmniConnectorBase]] = {}

    @classmethod
    def register(cls, name: str, ctor: Callable[[dict], OmniConnectorBase]):
        cls._registry[name] = ctor

    @classmethod
    def create(cls, spec: ConnectorSpec | dict | str) -> OmniConnectorBase:
        if isinstance(spec, str):
            spec = ConnectorSpec(spec)
        elif isinstance(spec, dict):
            spec = ConnectorSpec(spec.get("name", "SharedMemoryConnector"), dict(spec.get("extra", {})))
        if spec.name not in cls._registry:
            raise ValueError(f"unknown connector {spec.name!r}; registered: {sorted(cls._registry)}")
        c = cls._registry[spec.name](spec.extra)
        c.spec = {"name": spec.name, "extra": dict(spec.extra)}      # lets the receiving process open its own end
        return c


def _shm(cfg):
    from .shm_connector import SharedMemoryConnector
    return SharedMemoryConnector(cfg)


def _inproc(cfg):
    from .memory_connector import InProcConnector
    return InProcConnector(cfg)


def _device(cfg):
    from .device_connector import DeviceConnector
    return DeviceConnector(cfg)


def _mooncake(cfg):
    from .store_connectors import MooncakeConnector
    return MooncakeConnector(cfg)


def _yuanrong(cfg):
    from .store_connectors import YuanrongConnector
    return YuanrongConnector(cfg)


def _faulty(cfg):
    from .fault_injection import FaultInjectingConnector
    return FaultInjectingConnector(cfg)


OmniConnectorFactory.register("FaultInjectionConnector", _faulty)
OmniConnectorFactory.register("SharedMemoryConnector", _shm)
OmniConnectorFactory.register("InProcConnector", _inproc)
OmniConnectorFactory.register("DeviceConnector", _device)
OmniConnectorFactory.register("MooncakeConnector", _mooncake)
OmniConnectorFactory.register("YuanrongConnector", _yuanrong)


def load_omni_transfer_config(stage_configs: list, runtime_cfg: dict | None = None, default: str | None = None,
                              shm_threshold_bytes: int = 65536) -> dict[tuple[int, int], ConnectorSpec]:
    """One connector spec per pipeline edge.  Edges come from each stage's
    ``engine_input_source``; ``runtime.connectors`` + ``runtime.edges`` (or a stage's
    ``input_connectors``) override the default, which is shared memory for process-separated
    stages and the in-process connector otherwise."""
    runtime_cfg = runtime_cfg or {}
    named = {k: ConnectorSpec(v.get("name", k), dict(v.get("extra", {})))
             for k, v in (runtime_cfg.get("connectors") or {}).items()}
    edges: dict[tuple[int, int], ConnectorSpec] = {}
    for e in runtime_cfg.get("edges") or []:
        if e.get("connector"):              # an edge may only carry window settings
            edges[(int(e["from"]), int(e["to"]))] = named[e["connector"]]
    for sc in stage_configs:
        for src in sc.engine_input_source:
            key = (int(src), int(sc.stage_id))
            ic = (sc.input_connectors or {}).get(f"from_stage_{src}")
            if ic is not None:
                edges[key] = named[ic] if isinstance(ic, str) else ConnectorSpec(ic.get("name"), dict(ic.get("extra", {})))
            if key not in edges:
                name = default or ("SharedMemoryConnector" if sc.runtime.get("process") else "InProcConnector")
                edges[key] = ConnectorSpec(name, {"shm_threshold_bytes": shm_threshold_bytes})
    return edges


def initialize_orchestrator_connectors(stage_configs, runtime_cfg=None, **kw) -> dict[tuple[int, int], OmniConnectorBase]:
    specs = load_omni_transfer_config(stage_configs, runtime_cfg, **kw)
    return {edge: OmniConnectorFactory.create(spec) for edge, spec in specs.items()}
