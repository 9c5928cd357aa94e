"""Per-process KV-cache budget against a fake NVML (nothing here touches a real device)."""
import os
import types

from vllm_omni_b200.utils import gpu_memory as gm


class FakeNvml:
    def __init__(self, procs, fail_init=False):
        self.procs, self.fail_init, self.calls = procs, fail_init, []

    def nvmlInit(self):
        if self.fail_init:
            raise RuntimeError("no NVML")
        self.calls.append("init")

    def nvmlShutdown(self):
        self.calls.append("shutdown")

    def nvmlDeviceGetHandleByIndex(self, i):
        self.calls.append(("index", i))
        return ("h", i)

    def nvmlDeviceGetHandleByUUID(self, u):
        self.calls.append(("uuid", u))
        return ("h", u)

    def nvmlDeviceGetComputeRunningProcesses(self, h):
        return [types.SimpleNamespace(pid=p, usedGpuMemory=m) for p, m in self.procs]


def test_budget_uses_own_process_memory(monkeypatch):
    monkeypatch.delenv("CUDA_VISIBLE_DEVICES", raising=False)
    GiB = 1 << 30
    nv = FakeNvml([(os.getpid(), 30 * GiB), (4242, 60 * GiB)])
    # 180 GiB device, this stage may use 50 %, holds 30 GiB of weights; another stage holds 60 GiB
    assert gm.kv_cache_budget(180 * GiB, 85 * GiB, 0.5, nvml=nv) == 60 * GiB
    # never more than what is free right now
    assert gm.kv_cache_budget(180 * GiB, 20 * GiB, 0.5, nvml=nv) == 20 * GiB
    assert nv.calls[0] == "init" and nv.calls[-1] == "shutdown" and ("index", 0) in nv.calls


def test_budget_falls_back_without_nvml_or_pid(monkeypatch):
    GiB = 1 << 30
    assert gm.kv_cache_budget(100 * GiB, 70 * GiB, 0.6, nvml=FakeNvml([], fail_init=True)) == 30 * GiB
    assert gm.kv_cache_budget(100 * GiB, 70 * GiB, 0.6, nvml=FakeNvml([(1, 5 * GiB)])) == 30 * GiB   # pid not listed


def test_visible_devices_mapping(monkeypatch):
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "3,GPU-abc,5")
    assert gm.parse_cuda_visible_devices() == [3, "GPU-abc", 5]
    nv = FakeNvml([(os.getpid(), 7)])
    assert gm.process_gpu_memory(0, nvml=nv) == 7 and ("index", 3) in nv.calls
    assert gm.process_gpu_memory(1, nvml=nv) == 7 and ("uuid", "GPU-abc") in nv.calls
    assert gm.process_gpu_memory(9, nvml=nv) is None
