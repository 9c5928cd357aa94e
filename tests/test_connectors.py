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


def test_fault_injection_connector_drives_the_error_paths():
    """Scheduled host-side faults around a shared-memory connector: a dropped put is reported to the
    sender, a corrupted payload trips the receiver's checksum, a lost payload makes the adapter time
    out with a typed error, and an unfaulted transfer (with an injected delay) still arrives."""
    from vllm_omni_b200.connectors.adapter import try_recv_via_connector, try_send_via_connector
    c = OmniConnectorFactory.create({"name": "FaultInjectionConnector", "extra": {
        "inner": {"name": "SharedMemoryConnector", "extra": {"shm_threshold_bytes": 64, "get_retries": 2,
                                                             "get_retry_interval_s": 0.01}},
        # one schedule entry per connector call: put a, put b, get b, put c, get c, put d, get d
        "schedule": ["drop_put", "corrupt", None, None, None, None, "lose_get"], "delay_ms": 2}})
    data = {"h": torch.arange(64, dtype=torch.float32), "note": "x"}
    task = {}
    assert not try_send_via_connector(c, 0, 1, "a", data, task) and "connector_meta" not in task       # drop_put
    task = {}
    assert try_send_via_connector(c, 0, 1, "b", data, task)                                            # corrupt
    with pytest.raises(ValueError, match="checksum"):
        try_recv_via_connector(c, task)
    task = {}
    t0 = time.perf_counter()
    assert try_send_via_connector(c, 0, 1, "c", data, task)                                            # clean, delayed
    got = try_recv_via_connector(c, task)
    assert torch.equal(got["h"], data["h"]) and time.perf_counter() - t0 >= 0.004
    task = {}
    assert try_send_via_connector(c, 0, 1, "d", data, task)                                            # lost before the get
    with pytest.raises(TimeoutError, match="never arrived"):
        try_recv_via_connector(c, task)
    assert [f for f, _ in c.injected] == ["drop_put", "corrupt", "lose_get"]
    assert c.health()["injected_faults"] == 3
    c.cleanup_all()


def test_fault_rates_are_reproducible_and_kv_transfer_survives_drops():
    mk = lambda: OmniConnectorFactory.create({"name": "FaultInjectionConnector", "extra": {
        "inner": "InProcConnector", "rates": {"drop_put": 0.5}, "seed": 7}})
    a, b = mk(), mk()
    ra = [a.put(0, 1, f"k{i}", {"v": i})[0] for i in range(20)]
    rb = [b.put(0, 1, f"k{i}", {"v": i})[0] for i in range(20)]
    assert ra == rb and 3 < sum(ra) < 17
    # the KV sender retries with back-off until a put gets through
    conn = OmniConnectorFactory.create({"name": "FaultInjectionConnector", "extra": {
        "inner": "InProcConnector", "schedule": ["drop_put", "drop_put", None]}})
    send = OmniKVTransferManager.from_config({"stage_id": 0, "to_stages": [1], "need_send_cache": True,
                                              "send_retries": 4, "send_backoff_s": 0.001}, conn)
    req = Request("r1", [1, 2, 3], SamplingParams())
    assert send.handle_finished_requests_kv_transfer([req], _Runner()) == ["r1"] and send.stats["sent"] == 1
    assert [f for f, _ in conn.injected] == ["drop_put", "drop_put"]


def test_talker_prompt_length_follows_the_chat_turns():
    from vllm_omni_b200.connectors.adapter import compute_talker_prompt_ids_length as n
    IM, SYS, USR, AST = 151644, 8948, 872, 77091
    ids = [IM, SYS, 1, 2, 3, IM, USR, 4, 5, 6, 7, IM, AST, 8]
    assert n(ids) == 6 + 9                         # the user turn's six tokens + the nine-row assistant head
    assert n([IM, USR, 1, IM, AST, 2, 3, IM, USR, 4, 5, IM, AST, 6]) == 3 + 4 + 9      # the earlier assistant turn is dropped
    assert n([1, 2, 3]) == 0
