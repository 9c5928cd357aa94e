"""Decoder forward (dense and MoE) through the paged-KV path vs the plain fp32 restatement:
full prefill, chunked prefill with cached context, and token-by-token decode."""
import pytest
import torch

from vllm_omni_b200.models.qwen_decoder import (DecoderConfig, ModelBatch, PrefillSeg, QwenDecoderModel,
                                                reference_forward)


def _model(dtype, device, moe, head_dim=32):
    cfg = DecoderConfig(vocab_size=512, hidden_size=128, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, head_dim=head_dim, intermediate_size=256,
                        num_experts=8 if moe else 0, num_experts_per_tok=2, moe_intermediate_size=64)
    torch.manual_seed(0)
    m = QwenDecoderModel(cfg, dtype=dtype, device=device)
    for p in m.parameters():
        if p.dim() == 1:
            p.normal_(1.0, 0.1)
    return m


def _run_paged(m, ids, device, chunks, decode_from):
    """Prefill ids[:decode_from] in the given chunk sizes, then decode the rest token by token."""
    cfg = m.cfg
    bs, nb = 16, 32
    caches = [(torch.zeros(nb, bs, cfg.num_key_value_heads, cfg.head_dim, dtype=m.dtype_, device=device),
               torch.zeros(nb, bs, cfg.num_key_value_heads, cfg.head_dim, dtype=m.dtype_, device=device))
              for _ in range(cfg.num_hidden_layers)]
    table = torch.arange(3, 3 + (ids.numel() + bs - 1) // bs, dtype=torch.int32, device=device)
    assert int(table[-1]) < nb
    slot = lambda t: int(table[t // bs]) * bs + t % bs
    outs, done = [], 0
    for n in chunks:
        seg = PrefillSeg(0, n, done, table)
        b = ModelBatch(ids[done:done + n], torch.arange(done, done + n, device=device),
                       torch.tensor([slot(t) for t in range(done, done + n)], dtype=torch.int32, device=device), [seg])
        h, _ = m(b, caches)
        outs.append(h)
        done += n
    assert done == decode_from
    for t in range(decode_from, ids.numel()):
        b = ModelBatch(ids[t:t + 1], torch.tensor([t], device=device),
                       torch.tensor([slot(t)], dtype=torch.int32, device=device), [],
                       decode_rows=torch.tensor([0], device=device), decode_block_tables=table[None].contiguous(),
                       decode_seq_lens=torch.tensor([t + 1], dtype=torch.int32, device=device))
        h, _ = m(b, caches)
        outs.append(h)
    return torch.cat(outs, 0)


@pytest.mark.parametrize("moe", [False, True])
def test_decoder_paged_matches_reference_cpu(moe):
    m = _model(torch.float32, "cpu", moe)
    ids = torch.randint(0, 512, (40,))
    ref = reference_forward(m, ids)
    got = _run_paged(m, ids, "cpu", chunks=[17, 13], decode_from=30)
    assert torch.allclose(got, ref, atol=2e-4, rtol=1e-3), (got - ref).abs().max()


@pytest.mark.gpu
@pytest.mark.parametrize("moe", [False, True])
def test_decoder_paged_matches_reference_gpu(moe):
    dev = torch.device("cuda")
    m = _model(torch.bfloat16, dev, moe, head_dim=128)
    ids = torch.randint(0, 512, (300,), device=dev)
    ref = reference_forward(m, ids).float()
    got = _run_paged(m, ids, dev, chunks=[150, 140], decode_from=290).float()
    torch.cuda.synchronize()
    from vllm_omni_b200.ops import _native as nv
    assert int(nv.status_word(dev).item()) == 0
    # bf16 router logits can flip a near-tied expert for a few tokens (and everything after them in
    # the sequence sees that through attention), so judge the bulk of the rows, not the single worst
    row_err = (got - ref).abs().amax(-1)
    tol = 0.08 * max(1.0, ref.abs().max().item())
    if moe:
        assert row_err.median().item() < tol, row_err.median().item()
        assert torch.isfinite(got).all()
    else:
        assert row_err.max().item() < tol, row_err.max().item()


def _ep_worker(rank, world, backend, mode, dtype_name, head_dim, tol):
    """MoE decoder with the experts split over the ranks == all experts on one rank."""
    from vllm_omni_b200.parallel import parallel_state as ps
    dtype = getattr(torch, dtype_name)
    device = torch.device("cuda", rank) if backend == "nccl" else torch.device("cpu")
    ps.init_distributed_environment(world, rank, local_rank=rank, backend=backend)
    ps.initialize_model_parallel(tensor_parallel_size=world, backend=backend)     # the TP group doubles as EP group
    m = _model(dtype, device, True, head_dim=head_dim)
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 512, (150 if device.type == "cuda" else 40,), generator=g).to(device)
    ref = reference_forward(m, ids).float()
    m.enable_expert_parallel(ps.get_tp_group(), mode)
    assert m.layers[0].w13.shape[0] == 8 // world
    n = ids.numel()
    got = _run_paged(m, ids, device, chunks=[n // 2, n - n // 2 - 6], decode_from=n - 6).float()
    if device.type == "cuda":
        torch.cuda.synchronize()
        from vllm_omni_b200.ops import _native as nv
        assert int(nv.status_word(device).item()) == 0
        row_err = (got - ref).abs().amax(-1)
        assert row_err.median().item() < tol * max(1.0, ref.abs().max().item()), row_err.median().item()
        assert torch.isfinite(got).all()
    else:
        assert torch.allclose(got, ref, atol=tol, rtol=1e-3), (got - ref).abs().max()
    m.ep_reduce.close()
    ps.destroy_distributed_environment()


def test_expert_parallel_matches_single_rank_cpu_gloo():
    from dist_utils import run_distributed
    run_distributed(_ep_worker, 2, "gloo", args=("gloo", "nccl", "float32", 32, 3e-4))


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["nccl", "peer"])
def test_expert_parallel_matches_single_rank_gpu(mode):
    from dist_utils import run_distributed
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    run_distributed(_ep_worker, 2, "nccl", args=("nccl", mode, "bfloat16", 128, 0.08))
