"""Device-side waits give up instead of hanging: a barrier whose partner never arrives returns an
error status within its limit and leaves the context usable.  (The flag that would release the
wait is simply never written; nothing faults, traps or spins forever.)"""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def _barrier(lib, pages, rank, world, epoch, timeout_ns, status, nv):
    arr = (ctypes.c_void_p * world)(*[p.data_ptr() for p in pages])
    rc = lib.omni_peer_barrier(arr, ctypes.c_int(rank), ctypes.c_int(world), ctypes.c_void_p(epoch.data_ptr()),
                               ctypes.c_ulonglong(timeout_ns), nv.ptr(status), nv.stream_ptr())
    assert rc == 0


def test_barrier_wait_runs_out_and_reports():
    from vllm_omni_b200.ops import _native as nv
    dev = torch.device("cuda")
    lib = nv.lib("peer_rt")
    pages = [torch.zeros(16, dtype=torch.int64, device=dev) for _ in range(2)]     # both "ranks" on this GPU
    epoch = torch.zeros(1, dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    t0 = time.perf_counter()
    _barrier(lib, pages, 0, 2, epoch, 20_000_000, status, nv)      # rank 1 never enters: 20 ms limit
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert int(status.item()) == 5                                  # ERR_WAIT_PEER
    assert dt < 1.0
    assert int(epoch.item()) == 1 and int(pages[1][0].item()) == 1  # it did announce itself first
    # the context is still usable
    x = torch.arange(8, device=dev).float()
    assert float((x * 2).sum().item()) == 56.0


def test_barrier_completes_when_partner_has_arrived():
    from vllm_omni_b200.ops import _native as nv
    dev = torch.device("cuda")
    lib = nv.lib("peer_rt")
    pages = [torch.zeros(16, dtype=torch.int64, device=dev) for _ in range(2)]
    epochs = [torch.zeros(1, dtype=torch.int64, device=dev) for _ in range(2)]
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for step in range(3):
        # "rank 1" arrives first and gives up quickly (its partner has not come yet) ...
        scratch = torch.zeros(1, dtype=torch.int32, device=dev)
        _barrier(lib, pages, 1, 2, epochs[1], 1_000_000, scratch, nv)
        # ... so that rank 0 finds the flag already at this epoch and passes at once
        _barrier(lib, pages, 0, 2, epochs[0], 500_000_000, status, nv)
        torch.cuda.synchronize()
        assert int(status.item()) == 0 and int(epochs[0].item()) == step + 1


def _qkv_case(dev, B=1, S=256, H=4, D=128):
    torch.manual_seed(0)
    qkv = torch.randn(B, S, 3 * H * D, device=dev, dtype=torch.bfloat16)
    wq = torch.rand(D, device=dev, dtype=torch.bfloat16) + 0.5
    wk = torch.rand(D, device=dev, dtype=torch.bfloat16) + 0.5
    return qkv, wq, wk


def test_arrival_wait_inside_the_consumer_kernel_runs_out_and_reports():
    """The q/k-norm kernel waits for arrivals that no producer ever reports: it gives up after its
    limit, records ERR_WAIT_PEER and returns; the context stays usable."""
    from vllm_omni_b200.ops import _native as nv
    from vllm_omni_b200.ops import fused
    from vllm_omni_b200.parallel.peer_memory import SignalChannel
    dev = torch.device("cuda")
    nv.check_status(dev) if int(nv.status_word(dev).item()) == 0 else nv.status_word(dev).zero_()
    ch = SignalChannel(None, device=dev, timeout_ms=20)
    qkv, wq, wk = _qkv_case(dev)
    t0 = time.perf_counter()
    fused.qk_norm_rope_(qkv, 4, 4, 128, wq=wq, wk=wk, sync=ch.wait())
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    st = nv.status_word(dev)
    assert int(st.item()) == 5                                      # ERR_WAIT_PEER
    st.zero_()
    assert dt < 2.0
    assert int(ch.epoch[0].item()) == 1 and int(ch.epoch[1].item()) == 0     # the use was still accounted for
    x = torch.arange(8, device=dev).float()
    assert float((x * 2).sum().item()) == 56.0


def test_arrivals_reported_by_the_producer_release_the_consumer_every_use():
    """Single-rank channel: the GEMM reports an arrival when its stores are out, the q/k-norm kernel
    waits for it in-kernel; repeated uses (also replayed from a CUDA graph) keep the counters in step
    and the numbers equal to the unsynchronised path."""
    from vllm_omni_b200.ops import _native as nv
    from vllm_omni_b200.ops import fused, gemm
    from vllm_omni_b200.parallel.peer_memory import SignalChannel
    dev = torch.device("cuda")
    nv.status_word(dev).zero_()
    ch = SignalChannel(None, device=dev, timeout_ms=500)
    torch.manual_seed(1)
    H, D, S, K = 4, 128, 384, 256
    x = torch.randn(S, K, device=dev, dtype=torch.bfloat16)
    w = torch.randn(3 * H * D, K, device=dev, dtype=torch.bfloat16) * 0.05
    wq = torch.rand(D, device=dev, dtype=torch.bfloat16) + 0.5
    wk = torch.rand(D, device=dev, dtype=torch.bfloat16) + 0.5
    ref = gemm.linear(x, w).view(1, S, 3 * H * D).clone()
    fused.qk_norm_rope_(ref, H, H, D, wq=wq, wk=wk)
    out = torch.empty(1, S, 3 * H * D, device=dev, dtype=torch.bfloat16)

    def use():
        gemm.linear(x, w, out=out.view(S, -1), sync=ch.signal())
        fused.qk_norm_rope_(out, H, H, D, wq=wq, wk=wk, sync=ch.wait())
    for i in range(3):
        use()
        torch.cuda.synchronize()
        assert int(nv.status_word(dev).item()) == 0
        assert int(ch.counter.local[0].item()) == i + 1 and int(ch.epoch[0].item()) == i + 1
        assert torch.equal(out, ref)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        use()
    for i in range(3):
        out.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert int(nv.status_word(dev).item()) == 0
        assert torch.equal(out, ref)
    assert int(ch.counter.local[0].item()) == int(ch.epoch[0].item())
    assert int(ch.done[0].item()) == 0 and int(ch.epoch[1].item()) == 0
