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
