"""Ulysses sequence parallelism: sharded run == single-rank run.

CPU: 2 Gloo ranks exercise the layout logic through the all-to-all baseline mode.
GPU (needs 2 devices): the fused peer-memory path against the same single-rank result.
"""
import pytest
import torch

from dist_utils import run_distributed


def _build(dtype, device, head_dim, heads):
    from vllm_omni_b200.diffusion.models.qwen_image.transformer import (QwenImageTransformer2DModel,
                                                                        QwenImageTransformerConfig)
    axes = {32: (8, 12, 12), 128: (16, 56, 56)}[head_dim]
    cfg = QwenImageTransformerConfig(num_layers=2, attention_head_dim=head_dim, num_attention_heads=heads,
                                     joint_attention_dim=64, in_channels=16, out_channels=4, axes_dims_rope=axes)
    torch.manual_seed(0)
    m = QwenImageTransformer2DModel(cfg, dtype=dtype, device=device)
    g = torch.Generator(device="cpu").manual_seed(1)
    for p in m.parameters():
        if p.dim() == 1:
            p.copy_(torch.randn(p.shape, generator=g) * 0.5)
        else:
            p.copy_((torch.randn(p.shape, generator=g) * 0.02).to(p.dtype))
    return m


def _sp_worker(rank, world, backend, mode, dtype_name, head_dim, heads, tol, kind="ulysses"):
    from vllm_omni_b200.parallel import parallel_state as ps
    from vllm_omni_b200.parallel.ring import RingJointAttention
    from vllm_omni_b200.parallel.ulysses import UlyssesJointAttention
    dtype = getattr(torch, dtype_name)
    device = torch.device("cuda", rank) if backend == "nccl" else torch.device("cpu")
    ps.init_distributed_environment(world, rank, local_rank=rank, backend=backend)
    if kind == "ring":
        ps.initialize_model_parallel(sequence_parallel_size=world, ring_degree=world, backend=backend)
    else:
        ps.initialize_model_parallel(sequence_parallel_size=world, ulysses_degree=world, backend=backend)
    m = _build(dtype, device, head_dim, heads)
    B, h, w, St = 2, 8, 8, 6 * world
    g = torch.Generator(device="cpu").manual_seed(2)
    x = torch.randn(B, h * w, 16, generator=g).to(device)
    e = torch.randn(B, St, 64, generator=g).to(device)
    t = torch.tensor([0.6, 0.6], device=device)
    lens = [St, St - 3]
    ref = m(x, e, t, (1, h, w), txt_seq_lens=lens).float()
    if kind == "ring":
        m.sp = RingJointAttention(ps.get_sp_group().ring, heads, head_dim, mode=mode)
    else:
        m.sp = UlyssesJointAttention(ps.get_sp_group().ulysses, heads, head_dim, mode=mode)
    Si, Sl = h * w // world, St // world
    y = m(x[:, rank * Si:(rank + 1) * Si].contiguous(), e[:, rank * Sl:(rank + 1) * Sl].contiguous(), t, (1, h, w),
          txt_seq_lens=lens).float()
    if device.type == "cuda":
        torch.cuda.synchronize()
        from vllm_omni_b200.ops import _native as nv
        assert int(nv.status_word(device).item()) == 0
    err = (y - ref[:, rank * Si:(rank + 1) * Si]).abs().max().item()
    assert err < tol * max(1.0, ref.abs().max().item()), f"rank {rank}: {err}"
    m.sp.close()
    ps.destroy_distributed_environment()


def test_ulysses_matches_single_rank_cpu_gloo():
    run_distributed(_sp_worker, 2, "gloo", args=("gloo", "nccl", "float32", 32, 4, 2e-4))


def test_ring_matches_single_rank_cpu_gloo():
    run_distributed(_sp_worker, 2, "gloo", args=("gloo", "nccl", "float32", 32, 4, 2e-4, "ring"))


@pytest.mark.gpu
def test_ring_peer_kv_matches_single_rank_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    run_distributed(_sp_worker, 2, "nccl", args=("nccl", "peer", "bfloat16", 128, 4, 0.06, "ring"))


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["nccl", "fused"])
def test_ulysses_matches_single_rank_gpu(mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    run_distributed(_sp_worker, 2, "nccl", args=("nccl", mode, "bfloat16", 128, 4, 0.06))


def _tp_worker(rank, world, backend, mode, dtype_name, head_dim, heads, tol):
    """Tensor-parallel transformer (heads and MLP columns split over the ranks) == single rank."""
    from vllm_omni_b200.parallel import parallel_state as ps
    from vllm_omni_b200.parallel.tensor_parallel import shard_transformer
    dtype = getattr(torch, dtype_name)
    device = torch.device("cuda", rank) if backend == "nccl" else torch.device("cpu")
    ps.init_distributed_environment(world, rank, local_rank=rank, backend=backend)
    ps.initialize_model_parallel(tensor_parallel_size=world, backend=backend)
    m = _build(dtype, device, head_dim, heads)
    B, h, w, St = 2, 8, 8, 12
    g = torch.Generator(device="cpu").manual_seed(2)
    x = torch.randn(B, h * w, 16, generator=g).to(device)
    e = torch.randn(B, St, 64, generator=g).to(device)
    t = torch.tensor([0.6, 0.6], device=device)
    lens = [St, St - 3]
    ref = m(x, e, t, (1, h, w), txt_seq_lens=lens).float()
    shard_transformer(m, ps.get_tp_group(), mode)
    m._ws.key = None                      # the workspace is sized for this rank's share from here on
    y = m(x, e, t, (1, h, w), txt_seq_lens=lens).float()
    if device.type == "cuda":
        torch.cuda.synchronize()
        from vllm_omni_b200.ops import _native as nv
        assert int(nv.status_word(device).item()) == 0
    err = (y - ref).abs().max().item()
    assert err < tol * max(1.0, ref.abs().max().item()), f"rank {rank}: {err}"
    m.tp_reducer.close()
    ps.destroy_distributed_environment()


def test_tensor_parallel_matches_single_rank_cpu_gloo():
    run_distributed(_tp_worker, 2, "gloo", args=("gloo", "nccl", "float32", 32, 4, 2e-4))


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["nccl", "peer"])
def test_tensor_parallel_matches_single_rank_gpu(mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    run_distributed(_tp_worker, 2, "nccl", args=("nccl", mode, "bfloat16", 128, 4, 0.06))


def _hybrid_worker(rank, world, backend, mode, dtype_name, head_dim, heads, tol):
    """Ulysses 2 x ring 2 on four ranks == single rank."""
    from vllm_omni_b200.parallel import parallel_state as ps
    from vllm_omni_b200.parallel.hybrid import HybridJointAttention
    dtype = getattr(torch, dtype_name)
    device = torch.device("cuda", rank) if backend == "nccl" else torch.device("cpu")
    ps.init_distributed_environment(world, rank, local_rank=rank, backend=backend)
    ps.initialize_model_parallel(sequence_parallel_size=world, ulysses_degree=2, ring_degree=2, backend=backend)
    m = _build(dtype, device, head_dim, heads)
    B, h, w, St = 2, 8, 8, 6 * world
    g = torch.Generator(device="cpu").manual_seed(2)
    x = torch.randn(B, h * w, 16, generator=g).to(device)
    e = torch.randn(B, St, 64, generator=g).to(device)
    t = torch.tensor([0.6, 0.6], device=device)
    lens = [St, St - 7]                    # the second sample's padding spans more than one ring chunk
    ref = m(x, e, t, (1, h, w), txt_seq_lens=lens).float()
    m.sp = HybridJointAttention(ps.get_sp_group(), heads, head_dim, mode=mode)
    Si, Sl = h * w // world, St // world
    y = m(x[:, rank * Si:(rank + 1) * Si].contiguous(), e[:, rank * Sl:(rank + 1) * Sl].contiguous(), t, (1, h, w),
          txt_seq_lens=lens).float()
    if device.type == "cuda":
        torch.cuda.synchronize()
    err = (y - ref[:, rank * Si:(rank + 1) * Si]).abs().max().item()
    assert err < tol * max(1.0, ref.abs().max().item()), f"rank {rank}: {err}"
    m.sp.close()
    ps.destroy_distributed_environment()


def test_hybrid_ulysses_ring_matches_single_rank_cpu_gloo():
    run_distributed(_hybrid_worker, 4, "gloo", args=("gloo", "nccl", "float32", 32, 4, 2e-4))


@pytest.mark.gpu
def test_hybrid_ulysses_ring_matches_single_rank_gpu():
    import os
    if torch.cuda.device_count() < 4 or os.environ.get("OMNI_TEST_4GPU") != "1":
        pytest.skip("needs 4 GPUs and OMNI_TEST_4GPU=1 (the peer path of the hybrid has only run on CPU ranks so far)")
    run_distributed(_hybrid_worker, 4, "nccl", args=("nccl", "peer", "bfloat16", 128, 4, 0.06))


def _wan_sp_worker(rank, world, backend, uly, ring):
    """Wan-style video DiT with the token rows sharded over Ulysses x ring == single rank,
    including a sequence length that is not a multiple of the SP degree (padding + key mask)."""
    from vllm_omni_b200.diffusion.models.wan.transformer import WanTransformer3DModel, WanTransformerConfig
    from vllm_omni_b200.parallel import parallel_state as ps
    from vllm_omni_b200.parallel.sp_attention import SequenceParallelAttention
    ps.init_distributed_environment(world, rank, local_rank=rank, backend=backend)
    ps.initialize_model_parallel(sequence_parallel_size=world, ulysses_degree=uly, ring_degree=ring, backend=backend)
    cfg = WanTransformerConfig(num_layers=2, num_attention_heads=4, attention_head_dim=24, ffn_dim=128, text_dim=32,
                               freq_dim=32, in_channels=4, out_channels=4)
    torch.manual_seed(0)
    m = WanTransformer3DModel(cfg, dtype=torch.float32, device="cpu")
    g = torch.Generator().manual_seed(3)
    for T, H, W in ((2, 8, 8), (3, 6, 10)):            # 32 tokens (divisible) and 45 tokens (padded)
        x = torch.randn(1, 4, T, H, W, generator=g)
        e = torch.randn(1, 7, 32, generator=g)
        t = torch.tensor([500.0])
        m.sp = None
        ref = m(x, t, e)
        m.sp = SequenceParallelAttention(ps.get_sp_group(), 4, 24, mode="nccl")
        y = m(x, t, e)
        assert torch.allclose(y, ref, atol=3e-4, rtol=1e-3), (T, H, W, (y - ref).abs().max().item())
    ps.destroy_distributed_environment()


@pytest.mark.parametrize("uly,ring", [(2, 1), (1, 2), (2, 2)])
def test_wan_sequence_parallel_cpu_gloo(uly, ring):
    run_distributed(_wan_sp_worker, uly * ring, "gloo", args=("gloo", uly, ring))


def _zimage_sp_worker(rank, world, backend, uly, ring):
    """Z-Image-style single-stream DiT (joint image + text rows, per-sample text padding) with the
    rows sharded over the SP group == single rank."""
    from vllm_omni_b200.diffusion.models.z_image.transformer import ZImageTransformer2DModel, ZImageTransformerConfig
    from vllm_omni_b200.parallel import parallel_state as ps
    from vllm_omni_b200.parallel.sp_attention import SequenceParallelAttention
    ps.init_distributed_environment(world, rank, local_rank=rank, backend=backend)
    ps.initialize_model_parallel(sequence_parallel_size=world, ulysses_degree=uly, ring_degree=ring, backend=backend)
    cfg = ZImageTransformerConfig(dim=64, n_layers=2, n_refiner_layers=1, n_heads=4, n_kv_heads=4, in_channels=2,
                                  cap_feat_dim=24, axes_dims=(4, 6, 6), axes_lens=(128, 16, 16))
    torch.manual_seed(0)
    m = ZImageTransformer2DModel(cfg, dtype=torch.float32, device="cpu")
    g = torch.Generator().manual_seed(4)
    x = torch.randn(2, 6 * 5, 8, generator=g)
    e = torch.randn(2, 40, 24, generator=g)                # captions of 40 and 5 tokens -> 64 and 32 rows with pad tokens
    t = torch.tensor([0.3, 0.3])
    for lens in (None, [40, 5]):
        m.sp = None
        ref = m(x, e, t, (1, 6, 5), txt_seq_lens=lens)
        m.sp = SequenceParallelAttention(ps.get_sp_group(), 4, 16, mode="nccl")
        y = m(x, e, t, (1, 6, 5), txt_seq_lens=lens)
        assert torch.allclose(y, ref, atol=3e-4, rtol=1e-3), (lens, (y - ref).abs().max().item())
    ps.destroy_distributed_environment()


@pytest.mark.parametrize("uly,ring", [(2, 1), (2, 2)])
def test_zimage_sequence_parallel_cpu_gloo(uly, ring):
    run_distributed(_zimage_sp_worker, uly * ring, "gloo", args=("gloo", uly, ring))


def _spa_worker(rank, world, uly, ring, forced):
    """``SequenceParallelAttention`` in peer mode (pulled head exchange, gathered ring K/V, scatter epilogue)
    against one attention over the whole sequence; called twice so that buffers are reused."""
    import os
    from vllm_omni_b200.ops import _native as nv
    from vllm_omni_b200.ops.attention import attention_reference
    from vllm_omni_b200.parallel import parallel_state as ps
    from vllm_omni_b200.parallel.sp_attention import SequenceParallelAttention
    if forced:
        os.environ["OMNI_RING_MODE"] = forced
    dev = torch.device("cuda", rank)
    ps.init_distributed_environment(world, rank, local_rank=rank, backend="nccl")
    ps.initialize_model_parallel(sequence_parallel_size=world, ulysses_degree=uly, ring_degree=ring, backend="nccl")
    H, Dh, B, per = 4, 128, 2, 160
    S = per * world
    sp = SequenceParallelAttention(ps.get_sp_group(), H, Dh, mode="peer")
    for it, valid in enumerate((S, S - 37)):
        g = torch.Generator(device="cpu").manual_seed(7 + it)
        full = torch.randn(B, S, 3, H, Dh, generator=g).to(dev, torch.bfloat16)
        ref = attention_reference(full[:, :, 0].float(), full[:, :valid, 1].float(), full[:, :valid, 2].float())
        o = sp(full[:, rank * per:(rank + 1) * per].contiguous(), valid_len=None if valid == S else valid).float()
        torch.cuda.synchronize()
        assert int(nv.status_word(dev).item()) == 0
        err = (o - ref[:, rank * per:(rank + 1) * per]).abs().max().item()
        assert err < 0.03, f"rank {rank} uly {uly} ring {ring} valid {valid}: {err}"
    sp.close()
    ps.destroy_distributed_environment()


@pytest.mark.gpu
@pytest.mark.parametrize("uly,ring,forced", [(2, 1, None), (1, 2, "single"), (1, 2, "overlap")])
def test_single_stream_sp_attention_peer_mode_gpu(uly, ring, forced):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    run_distributed(_spa_worker, 2, "nccl", args=(uly, ring, forced))


@pytest.mark.gpu
@pytest.mark.parametrize("forced", ["single", "overlap"])
def test_single_stream_sp_attention_hybrid_gpu(forced):
    if torch.cuda.device_count() < 4:
        pytest.skip("needs 4 GPUs")
    run_distributed(_spa_worker, 4, "nccl", args=(2, 2, forced))
