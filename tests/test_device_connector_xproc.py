"""Device connector across processes: the producer pushes the payload into the consumer's arena
(own copy kernel over a CUDA IPC mapping); only a descriptor crosses the control plane.  Byte-exact
against the payload the producer built."""
import random

import pytest
import torch


def test_arena_ring_never_overlaps_and_never_wedges():
    from vllm_omni_b200.connectors.device_connector import ArenaRing
    own = ArenaRing("omni_dc_test_ring", create=True, arena_bytes=4096, handle=b"h" * 64)
    peer = ArenaRing("omni_dc_test_ring", create=False)
    try:
        assert peer.ready and peer.arena_bytes == 4096 and peer.handle == b"h" * 64
        live, rng, made = {}, random.Random(0), 0
        for _ in range(6000):
            if live and (rng.random() < 0.5 or len(live) > 6):
                e = rng.choice(list(live))
                own.release(e)                       # the consumer frees in any order
                del live[e]
            n = rng.choice([100, 256, 700, 1024, 1500])
            got = peer.reserve(n)
            if got is None:
                assert live, "an empty arena must always take a payload that fits"
                continue
            e, off = got
            size = (n + 255) // 256 * 256
            assert off % 256 == 0 and off + size <= 4096
            for o2, s2 in live.values():
                assert off + size <= o2 or o2 + s2 <= off
            live[e] = (off, size)
            made += 1
        assert made > 2000
        with pytest.raises(ValueError):
            peer.reserve(8192)
    finally:
        peer.close()
        own.close()


def _payload(dev, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return {"hidden": torch.randn(37, 2048, generator=g).to(dev, torch.bfloat16),
            "kv": [(torch.randn(5, 16, 4, 128, generator=g).to(dev, torch.bfloat16),
                    torch.randn(5, 16, 4, 128, generator=g).to(dev, torch.bfloat16)) for _ in range(2)],
            "codes": torch.randint(0, 1000, (16, 33), generator=g).to(dev),
            "lens": torch.tensor([3, 5, 7]), "tag": "x", "odd": torch.arange(13, dtype=torch.uint8).to(dev)}


def _producer(dev_index, q_desc, n_rounds):
    from vllm_omni_b200.connectors.device_connector import DeviceConnector
    torch.cuda.set_device(dev_index)
    dev = torch.device("cuda", dev_index)
    c = DeviceConnector({"cross_process": True, "name": "omni_dc_test", "arena_mb": 8, "get_timeout_s": 20})
    for i in range(n_rounds):
        ok, nbytes, meta = c.put(0, 1, f"req{i}", _payload(dev, 100 + i))
        assert ok and nbytes > 0
        q_desc.put(meta)
    q_desc.put(None)
    import time
    time.sleep(1.0)                # keep the mapping alive until the consumer has drained
    c.close()


@pytest.mark.gpu
def test_cross_process_put_get_is_byte_exact():
    import torch.multiprocessing as mp
    from vllm_omni_b200.connectors.device_connector import DeviceConnector
    n_dev = torch.cuda.device_count()
    cons_dev, prod_dev = (1, 0) if n_dev >= 2 else (0, 0)
    prev_dev = torch.cuda.current_device()
    torch.cuda.set_device(cons_dev)
    c = DeviceConnector({"cross_process": True, "name": "omni_dc_test", "arena_mb": 8})
    c.open_receiver(0, 1)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    rounds = 12                                        # more than the arena holds at once: ranges are recycled
    p = ctx.Process(target=_producer, args=(prod_dev, q, rounds))
    p.start()
    try:
        i = 0
        while True:
            meta = q.get(timeout=120)
            if meta is None:
                break
            got, nbytes = c.get(0, 1, f"req{i}", meta)
            want = _payload(torch.device("cuda", cons_dev), 100 + i)
            assert got["tag"] == "x" and torch.equal(got["lens"], want["lens"])
            assert torch.equal(got["hidden"], want["hidden"]) and got["hidden"].device.index == cons_dev
            assert torch.equal(got["codes"], want["codes"]) and torch.equal(got["odd"], want["odd"])
            for (k1, v1), (k2, v2) in zip(got["kv"], want["kv"]):
                assert torch.equal(k1, k2) and torch.equal(v1, v2)
            i += 1
        assert i == rounds
    finally:
        p.join(30)
        if p.is_alive():
            p.terminate()
        c.close()
        torch.cuda.set_device(prev_dev)
    assert p.exitcode == 0
