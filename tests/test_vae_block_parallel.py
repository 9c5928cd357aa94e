"""VAE block decode across ranks: one core block per rank decoded with a latent halo; with a decoder
whose receptive field fits inside the halo the stitched image equals the single-rank decode exactly."""
import types

import pytest
import torch
from torch import nn

from dist_utils import run_distributed
from vllm_omni_b200.parallel.vae_patch_parallel import VaePatchParallelism, block_bounds, grid_for


def test_grid_and_block_bounds():
    assert grid_for(1) == (1, 1) and grid_for(2) == (1, 2) and grid_for(4) == (2, 2) and grid_for(6) == (2, 3) and grid_for(8) == (2, 4)
    cover = torch.zeros(10, 13)
    for i in range(6):
        (h0, h1, w0, w1), (p0, p1, q0, q1) = block_bounds(10, 13, 2, 3, i, 2)
        cover[h0:h1, w0:w1] += 1
        assert p0 <= h0 and p1 >= h1 and q0 <= w0 and q1 >= w1 and p0 >= 0 and p1 <= 10 and q1 <= 13
        assert (h0 - p0 >= 2 or p0 == 0) and (p1 - h1 >= 2 or p1 == 10)
    assert (cover == 1).all()


class _ToyVae(nn.Module):
    """Two 3x3 convolutions and a 2x nearest up-sampling: receptive field 2 latent pixels each way."""

    def __init__(self):
        super().__init__()
        g = torch.Generator().manual_seed(3)
        self.c1, self.c2 = nn.Conv2d(4, 8, 3, padding=1), nn.Conv2d(8, 3, 3, padding=1)
        for p in self.parameters():
            p.data = torch.randn(p.shape, generator=g) * 0.2
        self.cfg = types.SimpleNamespace(spatial_scale=2)
        self.dtype = torch.float32
        self.post_quant_conv = nn.Identity()

    def denormalize(self, z):
        return z

    def decoder(self, z):
        return self.c2(torch.nn.functional.interpolate(torch.relu(self.c1(z)), scale_factor=2, mode="nearest")) * 0.1

    def decode(self, z):
        return self.decoder(z).clamp(-1, 1)


def _worker(rank, world, backend="gloo"):
    from vllm_omni_b200.parallel import parallel_state as ps
    dev = torch.device("cuda", rank) if backend == "nccl" else torch.device("cpu")
    ps.init_distributed_environment(world_size=world, rank=rank, local_rank=rank, backend=backend)
    ps.initialize_model_parallel(vae_patch_parallel_size=world, data_parallel_size=world, backend=backend)
    vae = _ToyVae().to(dev)
    pipe = types.SimpleNamespace(vae=vae, vae_decode=None)
    vp = VaePatchParallelism(pipe, world, tile_latent=64, overlap=8).install()
    z = torch.randn(2, 4, 12, 16, generator=torch.Generator().manual_seed(0)).to(dev)
    want = vae.decode(z)
    for _ in range(2):                    # the second call reuses the peer image after the barrier
        got = pipe.vae_decode(z)
        assert got.shape == want.shape == (2, 3, 24, 32)
        assert (got - want).abs().max().item() < (1e-5 if backend == "gloo" else 2e-3)      # cuDNN may pick TF32-free but differently ordered sums per block shape
    if backend == "nccl":
        assert vp._img is not None        # the device path (blocks stored into every rank's image through peer memory) ran
    vp.close()
    ps.destroy_distributed_environment()


@pytest.mark.parametrize("world", [2, 4])
def test_block_decode_with_halo_equals_single_rank(world):
    run_distributed(_worker, world)


@pytest.mark.gpu
def test_block_decode_peer_stores_two_gpus():
    """The device path: every rank stores its core block into the image buffer of every rank with the pitched
    peer copy kernel, two barriers around the stores."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    run_distributed(_worker, 2, "nccl", args=("nccl",))
