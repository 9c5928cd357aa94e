"""Chunk streaming between stage engines through a connector
(vllm_omni/distributed/omni_connectors/transfer_adapter/{base,chunk_transfer_adapter}.py).

A producer stage saves chunks under ``{request}_{stage}_{chunk}``; a consumer request sits in
``WAITING_FOR_CHUNK`` until its next chunk arrives, then the adapter appends the chunk to the
request's prompt (token ids + embeddings) and the scheduler picks it up.  The last chunk is
flagged.  ``poll`` is called by the scheduler each step and never blocks; ``save_async``
enqueues on a sender thread so the engine step does not wait on the connector.
"""
from __future__ import annotations

import queue
import threading

import torch

from ..logger import init_logger
from .factory import OmniConnectorFactory

logger = init_logger(__name__)


class OmniTransferAdapterBase:
    def __init__(self, connector, stage_id: int, start_threads: bool = True):
        self.connector = connector
        self.stage_id = stage_id
        self._lock = threading.Lock()
        self._send_q: queue.Queue = queue.Queue()
        self._stop = threading.Event()
        self._sender = None
        if start_threads:
            self._sender = threading.Thread(target=self._send_loop, name=f"chunk-sender-{stage_id}", daemon=True)
            self._sender.start()

    def _send_loop(self):
        while not self._stop.is_set():
            try:
                item = self._send_q.get(timeout=0.05)
            except queue.Empty:
                continue
            self._do_send(*item)

    def _do_send(self, to_stage, key, payload):
        ok, _, _ = self.connector.put(self.stage_id, to_stage, key, payload)
        if not ok:
            logger.error("chunk %s to stage %s could not be stored", key, to_stage)

    def close(self):
        self._stop.set()
        if self._sender is not None:
            self._sender.join(timeout=1)


class OmniChunkTransferAdapter(OmniTransferAdapterBase):
    def __init__(self, connector, stage_id: int, from_stage: int | None = None, to_stage: int | None = None,
                 start_threads: bool = True):
        super().__init__(connector, stage_id, start_threads)
        self.from_stage = stage_id - 1 if from_stage is None else from_stage
        self.to_stage = stage_id + 1 if to_stage is None else to_stage
        self._next_chunk: dict[str, int] = {}       # consumer side: next chunk index per request
        self._sent_chunks: dict[str, int] = {}      # producer side

    @classmethod
    def from_spec(cls, spec: dict, stage_id: int, model_stage: str | None = None):
        conn = spec.get("connector_obj") or OmniConnectorFactory.create(spec.get("connector", spec))
        return cls(conn, stage_id, spec.get("from_stage"), spec.get("to_stage"))

    @staticmethod
    def chunk_key(request_id: str, stage_id: int, idx: int) -> str:
        return f"{request_id}_{stage_id}_{idx}"

    # ------------------------------------------------------------------ producer
    def save_async(self, request_id: str, payload: dict, last: bool = False, sync: bool = False) -> int:
        idx = self._sent_chunks.get(request_id, 0)
        self._sent_chunks[request_id] = idx + 1
        payload = dict(payload, last=bool(last), chunk_index=idx)
        key = self.chunk_key(request_id, self.stage_id, idx)
        if sync or self._sender is None:
            self._do_send(self.to_stage, key, payload)
        else:
            self._send_q.put((self.to_stage, key, payload))
        if last:
            self._sent_chunks.pop(request_id, None)
        return idx

    # ------------------------------------------------------------------ consumer
    def poll(self, req) -> bool:
        """Non-blocking: pull every chunk that has arrived for ``req``.  Returns True when at least
        one chunk was appended."""
        got = False
        while req.expects_more_chunks:
            idx = self._next_chunk.get(req.request_id, 0)
            key = self.chunk_key(req.request_id, self.from_stage, idx)
            res = self._try_get(key)
            if res is None:
                break
            payload = res[0]
            self._next_chunk[req.request_id] = idx + 1
            ids = list(payload.get("token_ids") or [])
            emb = payload.get("embeds")
            if emb is None and "thinker_embeddings" in payload:
                emb = payload["thinker_embeddings"]
            if not ids and emb is not None:
                ids = [0] * emb.shape[0]
            for k, v in payload.items():
                if k not in ("token_ids", "embeds", "last", "chunk_index"):
                    prev = req.additional_information.get(k)
                    if isinstance(v, torch.Tensor) and isinstance(prev, torch.Tensor) and prev.dim() == v.dim():
                        req.additional_information[k] = torch.cat([prev, v], 0)
                    else:
                        req.additional_information[k] = v
            req.append_prompt_chunk(ids, emb, last=bool(payload.get("last")))
            got = True
            if payload.get("last"):
                self._next_chunk.pop(req.request_id, None)
        return got

    def _try_get(self, key):
        c = self.connector
        # a non-blocking probe: connectors retry internally, so ask for a single attempt
        old = (getattr(c, "retries", None), getattr(c, "get_timeout", None))
        try:
            if old[0] is not None:
                c.retries = 1
            if old[1] is not None:
                c.get_timeout = 0.0
            return c.get(self.from_stage, self.stage_id, key, None)
        finally:
            if old[0] is not None:
                c.retries = old[0]
            if old[1] is not None:
                c.get_timeout = old[1]
