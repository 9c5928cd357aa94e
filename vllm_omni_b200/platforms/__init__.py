"""Platform layer.  The reference detects cuda / rocm / npu / xpu and dispatches through an
``OmniPlatform`` interface (vllm_omni/platforms/__init__.py, interface.py).  This framework
targets one platform — NVIDIA Blackwell, sm_100a — so the interface is kept (callers and
plugins can query it) but there is exactly one implementation and no backend dispatch."""
from __future__ import annotations

import torch


class OmniPlatform:
    device_type = "cuda"
    dist_backend = "nccl"
    device_control_env_var = "CUDA_VISIBLE_DEVICES"

    @staticmethod
    def is_available() -> bool:
        return torch.cuda.is_available()

    @staticmethod
    def device_count() -> int:
        return torch.cuda.device_count() if torch.cuda.is_available() else 0

    @staticmethod
    def get_device_capability(idx: int = 0):
        return torch.cuda.get_device_capability(idx) if torch.cuda.is_available() else None

    @classmethod
    def check_supported(cls) -> None:
        """The native kernels are sm_100a only (tcgen05 / TMEM): refuse other GPUs loudly."""
        if torch.cuda.is_available():
            cc = torch.cuda.get_device_capability(0)
            if cc[0] != 10:
                raise RuntimeError(f"vllm_omni_b200 needs a Blackwell (sm_100a) GPU, found compute capability {cc}")

    @staticmethod
    def get_attention_backend() -> str:
        return "TCGEN05_FLASH"

    @staticmethod
    def mem_get_info(idx: int = 0):
        return torch.cuda.mem_get_info(idx)

    @staticmethod
    def synchronize():
        if torch.cuda.is_available():
            torch.cuda.synchronize()


class CpuPlatform(OmniPlatform):
    """PyTorch restatement path (tests, the tiny configuration)."""
    device_type = "cpu"
    dist_backend = "gloo"


current_omni_platform = OmniPlatform() if torch.cuda.is_available() else CpuPlatform()
