"""Failure detection of the multi-process diffusion executor, with the failures made on the host:
a worker process that is killed, one that is frozen (SIGSTOP) and a call that overruns its
time limit.  The worker runs the tiny pipeline on the CPU; no GPU is involved."""
import os
import signal
import time

import pytest
import torch

from vllm_omni_b200.diffusion.data import OmniDiffusionConfig
from vllm_omni_b200.diffusion.executor import MultiprocDiffusionExecutor, WorkerDeadError


def _config():
    return OmniDiffusionConfig.from_kwargs(model="TinyMMDiTPipeline", model_class_name="TinyMMDiTPipeline",
                                           dtype=torch.float32, device="cpu", distributed_executor_backend="mp")


@pytest.fixture()
def executor():
    ex = MultiprocDiffusionExecutor(_config(), init_timeout=120, heartbeat_stall_s=1.5)
    yield ex
    for p in list(ex.procs):
        if p.is_alive():
            try:
                os.kill(p.pid, signal.SIGCONT)
            except OSError:
                pass
    ex.shutdown()


def test_rpc_roundtrip_then_killed_worker_is_reported(executor):
    assert executor.check_health()
    assert executor.collective_rpc("list_loras", timeout=30) == []
    os.kill(executor.procs[0].pid, signal.SIGKILL)
    executor.procs[0].join(10)
    assert not executor.check_health()
    with pytest.raises(WorkerDeadError, match="died"):
        executor.collective_rpc("list_loras", timeout=30)


def test_frozen_worker_is_detected_by_missing_heartbeats(executor):
    assert executor.collective_rpc("check_health", timeout=30) is True
    os.kill(executor.procs[0].pid, signal.SIGSTOP)          # alive for the OS, but makes no progress
    t0 = time.monotonic()
    with pytest.raises(WorkerDeadError, match="stopped responding"):
        executor.collective_rpc("list_loras", timeout=60)
    assert time.monotonic() - t0 < 10
    assert executor.check_health()                           # process exists: only the heartbeat tells
    os.kill(executor.procs[0].pid, signal.SIGCONT)


def test_rpc_time_limit(executor):
    executor.heartbeat_stall_s = 60.0                        # the call's own limit must fire first
    os.kill(executor.procs[0].pid, signal.SIGSTOP)
    with pytest.raises(TimeoutError):
        executor.collective_rpc("list_loras", timeout=1.0)
    os.kill(executor.procs[0].pid, signal.SIGCONT)
    # the late reply of the timed-out call must not be taken for the next call's answer
    assert executor.collective_rpc("check_health", timeout=30) is True
