"""KV-cache hand-off between stages (Bagel pattern: an AR stage prefills, a DiT stage consumes
the KV as ``past_key_values``; vllm_omni/distributed/omni_connectors/kv_transfer_manager.py:
47-459).

Sender: after the scheduler marks a request (``prefill_finished`` / ``special_token``), the
runner gathers the request's pages into contiguous per-layer tensors and puts them in the
connector under ``kv_{request_id}``; the put is retried with exponential backoff and the
scheduler frees the pages only after this manager reports the request as extracted.
Receiver: polls the connector (0.5 s period, 30 s timeout by default) and attaches the tensors
to the request's sampling parameters.  With a device-capable connector the tensors never
leave GPU memory.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field

import torch

from ..logger import init_logger
from .factory import OmniConnectorFactory

logger = init_logger(__name__)


@dataclass
class OmniKVCacheConfig:
    connector: dict = field(default_factory=lambda: {"name": "InProcConnector"})
    stage_id: int = 0
    from_stage: int | None = None
    to_stages: list[int] = field(default_factory=list)
    need_send_cache: bool = False
    need_recv_cache: bool = False
    kv_transfer_criteria: dict = field(default_factory=dict)
    recv_timeout_s: float = 30.0
    recv_poll_s: float = 0.5
    send_retries: int = 3
    send_backoff_s: float = 0.05


class OmniKVTransferManager:
    def __init__(self, cfg: OmniKVCacheConfig, connector=None):
        self.cfg = cfg
        self.connector = connector or OmniConnectorFactory.create(cfg.connector)
        self.stats = {"sent": 0, "received": 0, "send_failures": 0, "recv_timeouts": 0, "bytes": 0}

    @classmethod
    def from_config(cls, d: dict, connector=None) -> "OmniKVTransferManager":
        names = set(OmniKVCacheConfig.__dataclass_fields__)
        return cls(OmniKVCacheConfig(**{k: v for k, v in d.items() if k in names}), connector)

    @staticmethod
    def key(request_id: str) -> str:
        return f"kv_{request_id}"

    # ------------------------------------------------------------------ sender
    def handle_finished_requests_kv_transfer(self, requests, runner) -> list[str]:
        """Extract + send the KV of ``requests``; returns the ids whose pages may be freed."""
        done = []
        if not self.cfg.need_send_cache:
            return [r.request_id for r in requests]
        for req in requests:
            payload = runner.extract_kv(req)
            data = {"request_id": req.request_id, "num_tokens": payload["num_tokens"],
                    "layers": [(k, v) for (k, v) in payload["layers"]],
                    "prompt_token_ids": list(req.prompt_token_ids)}
            if self._send_with_retry(req.request_id, data):
                done.append(req.request_id)
                self.stats["sent"] += 1
            else:
                self.stats["send_failures"] += 1
                logger.error("KV transfer for %s failed after %d attempts", req.request_id, self.cfg.send_retries)
                done.append(req.request_id)      # free the pages anyway; the consumer will time out
        return done

    def _send_with_retry(self, request_id: str, data) -> bool:
        delay = self.cfg.send_backoff_s
        targets = self.cfg.to_stages or [self.cfg.stage_id + 1]
        for attempt in range(max(1, self.cfg.send_retries)):
            ok_all = True
            for to in targets:
                ok, size, _ = self.connector.put(self.cfg.stage_id, to, self.key(request_id), data)
                ok_all &= bool(ok)
                if ok:
                    self.stats["bytes"] += size
            if ok_all:
                return True
            time.sleep(delay)
            delay *= 2
        return False

    # ------------------------------------------------------------------ receiver
    def receive_kv_cache(self, req, target_device=None) -> bool:
        """Blocks (bounded) until the KV for the request arrives; attaches it to
        ``req.sampling_params.past_key_values``."""
        if not self.cfg.need_recv_cache:
            return False
        rid = req.request_ids[0] if getattr(req, "request_ids", None) else getattr(req, "request_id", "")
        src = self.cfg.from_stage if self.cfg.from_stage is not None else self.cfg.stage_id - 1
        deadline = time.monotonic() + self.cfg.recv_timeout_s
        while True:
            res = self.connector.get(src, self.cfg.stage_id, self.key(rid), None)
            if res is not None:
                data, size = res
                self.apply_kv_cache_to_request(req, data, target_device)
                self.stats["received"] += 1
                self.stats["bytes"] += size
                return True
            if time.monotonic() >= deadline:
                self.stats["recv_timeouts"] += 1
                logger.warning("timed out waiting for KV of %s", rid)
                return False
            time.sleep(self.cfg.recv_poll_s)

    @staticmethod
    def apply_kv_cache_to_request(req, data, target_device=None) -> None:
        layers = data["layers"]
        if target_device is not None:
            layers = [(k.to(target_device, non_blocking=True), v.to(target_device, non_blocking=True)) for k, v in layers]
        sp = req.sampling_params
        sp.past_key_values = layers
        sp.kv_metadata = {"num_tokens": data["num_tokens"], "prompt_token_ids": data.get("prompt_token_ids")}
