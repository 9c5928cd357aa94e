"""CFG parallelism: two ranks exchange their velocity predictions and both end the step with the
latents a single rank would compute (guidance mix, optional norm rescale, Euler update)."""
import pytest
import torch

from dist_utils import run_distributed


def _cfg_worker(rank, world, backend):
    from vllm_omni_b200.ops import fused
    from vllm_omni_b200.parallel import parallel_state as ps
    from vllm_omni_b200.parallel.cfg_parallel import CFGExchange
    device = torch.device("cuda", rank) if backend == "nccl" else torch.device("cpu")
    ps.init_distributed_environment(world, rank, local_rank=rank, backend=backend)
    ps.initialize_model_parallel(cfg_parallel_size=2, backend=backend)
    ex = CFGExchange(ps.get_cfg_group())
    g = torch.Generator(device="cpu").manual_seed(5)
    dt = torch.bfloat16 if device.type == "cuda" else torch.float32
    lat = torch.randn(2, 96, 64, generator=g).to(device)
    ref = lat.clone()
    for step in range(3):                      # three steps: both parities of the double buffer
        pos = torch.randn(2, 96, 64, generator=g).to(device, dt)
        neg = torch.randn(2, 96, 64, generator=g).to(device, dt)
        ref = fused.cfg_euler_step_reference(pos, neg, ref, 4.0, -0.05, step != 1)
        ex.step(pos if rank == 0 else neg, lat, 4.0, -0.05, step != 1)
    if device.type == "cuda":
        torch.cuda.synchronize()
        from vllm_omni_b200.ops import _native as nv
        assert int(nv.status_word(device).item()) == 0
    assert (lat - ref).abs().max().item() < (2e-2 if device.type == "cuda" else 1e-5)
    ex.close()
    ps.destroy_distributed_environment()


def test_cfg_exchange_cpu_gloo():
    run_distributed(_cfg_worker, 2, "gloo", args=("gloo",))


@pytest.mark.gpu
def test_cfg_exchange_peer_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    run_distributed(_cfg_worker, 2, "nccl", args=("nccl",))
