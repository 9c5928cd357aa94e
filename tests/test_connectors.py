"""Connector data plane on CPU tensors: serialisation, shm, fault injection (dropped payloads,
corrupt checksum), KV transfer with retries / time-outs, chunk streaming state machine."""
import time

import pytest
import torch

from vllm_omni_b200.connectors.chunk_transfer_adapter import OmniChunkTransferAdapter
from vllm_omni_b200.connectors.factory import OmniConnectorFactory
from vllm_omni_b200.connectors.kv_transfer_manager import OmniKVTransferManager
from vllm_omni_b200.connectors.memory_connector import InProcConnector
from vllm_omni_b200.connectors.shm_connector import SharedMemoryConnector
from vllm_omni_b200.engine.request import Request, RequestStatus
from vllm_omni_b200.inputs import OmniDiffusionSamplingParams, SamplingParams


def test_shm_roundtrip_and_checksum_fault():
    c = SharedMemoryConnector({"shm_threshold_bytes": 64, "get_retries": 2, "get_retry_interval_s": 0.01})
    data = {"h": torch.randn(4, 8).bfloat16(), "ids": [1, 2, 3]}
    ok, n, meta = c.put(0, 1, "r", data)
    assert ok and "shm" in meta
    bad = dict(meta, crc=meta["crc"] ^ 1)                 # corrupted in flight
    with pytest.raises(ValueError):
        c.get(0, 1, "r", bad)
    ok, n, meta = c.put(0, 1, "r2", data)
    got, n2 = c.get(0, 1, "r2", meta)
    assert n2 == n and torch.equal(got["h"], data["h"]) and got["ids"] == [1, 2, 3]
    assert c.get(0, 1, "missing", {"shm": {"name": "nope_does_not_exist", "size": 1}}) is None   # dropped payload
    c.cleanup_all()


def test_factory_and_store_connectors_fail_clearly():
    assert isinstance(OmniConnectorFactory.create("InProcConnector"), InProcConnector)
    with pytest.raises(ValueError):
        OmniConnectorFactory.create("NoSuchConnector")
    with pytest.raises(RuntimeError, match="mooncake"):
        OmniConnectorFactory.create({"name": "MooncakeConnector"})


class _FlakyConnector(InProcConnector):
    def __init__(self, fail_first):
        super().__init__({"get_timeout_s": 0.05})
        self.fail_first, self.attempts = fail_first, 0

    def put(self, *a):
        self.attempts += 1
        if self.attempts <= self.fail_first:
            return False, 0, None
        return super().put(*a)


class _Runner:
    def extract_kv(self, req):
        return {"num_tokens": 3, "layers": [(torch.ones(3, 2, 4), torch.zeros(3, 2, 4)) for _ in range(2)]}


def test_kv_transfer_retry_then_receive():
    conn = _FlakyConnector(fail_first=2)
    send = OmniKVTransferManager.from_config({"stage_id": 0, "to_stages": [1], "need_send_cache": True,
                                              "send_retries": 4, "send_backoff_s": 0.001}, conn)
    req = Request("q1", [1, 2, 3], SamplingParams())
    assert send.handle_finished_requests_kv_transfer([req], _Runner()) == ["q1"]
    assert conn.attempts == 3 and send.stats["sent"] == 1
    recv = OmniKVTransferManager.from_config({"stage_id": 1, "from_stage": 0, "need_recv_cache": True,
                                              "recv_timeout_s": 0.2, "recv_poll_s": 0.01}, conn)

    class DReq:
        request_ids = ["q1"]
        sampling_params = OmniDiffusionSamplingParams()
    d = DReq()
    assert recv.receive_kv_cache(d) and len(d.sampling_params.past_key_values) == 2
    assert d.sampling_params.kv_metadata["num_tokens"] == 3
    d2 = DReq()
    d2.request_ids = ["never-sent"]
    t = time.monotonic()
    assert not recv.receive_kv_cache(d2) and recv.stats["recv_timeouts"] == 1
    assert time.monotonic() - t < 2.0


def test_chunk_adapter_state_machine():
    conn = InProcConnector({"get_timeout_s": 0.0})
    prod = OmniChunkTransferAdapter(conn, stage_id=0, to_stage=1, start_threads=False)
    cons = OmniChunkTransferAdapter(conn, stage_id=1, from_stage=0, start_threads=False)
    req = Request("c1", [], SamplingParams(), expects_more_chunks=True)
    req.status = RequestStatus.WAITING_FOR_CHUNK
    assert not cons.poll(req) and req.status == RequestStatus.WAITING_FOR_CHUNK
    prod.save_async("c1", {"token_ids": [5, 6], "embeds": torch.ones(2, 4)}, sync=True)
    assert cons.poll(req)
    assert req.status == RequestStatus.WAITING and req.prompt_token_ids == [5, 6] and req.expects_more_chunks
    prod.save_async("c1", {"token_ids": [7], "embeds": torch.zeros(1, 4)}, last=True, sync=True)
    assert cons.poll(req)
    assert req.prompt_token_ids == [5, 6, 7] and req.prompt_embeds.shape == (3, 4) and not req.expects_more_chunks
    assert not cons.poll(req)
