"""Tensor- and expert-parallel AR stages: every rank runs the same engine on its shard of the
decoder; greedy tokens equal the single-rank run.  CPU: two Gloo ranks (rank 1 is spawned by rank 0)."""
import pytest
import torch

from vllm_omni_b200.inputs import SamplingParams

PROMPTS = [{"prompt_token_ids": [506, 509, 11, 12, 507, 506, 510, 13]},
           {"prompt_token_ids": [506, 509, 20, 507, 506, 510]},
           {"prompt_token_ids": [3, 4, 5, 6, 7, 8, 9, 10, 11]}]


def _run(arch, tp, ep=False, device="cpu", overrides=None, max_tokens=8):
    from vllm_omni_b200.entrypoints.omni_llm import OmniLLM
    ov = dict(overrides or {"tiny": True, "vocab_size": 600})
    ov["moe"] = "Moe" in arch
    llm = OmniLLM(None, model_arch=arch, device=device, num_gpu_blocks=64, block_size=4 if device == "cpu" else 16,
                  tensor_parallel_size=tp, enable_expert_parallel=ep, model_overrides=ov)
    try:
        sp = SamplingParams(temperature=0.0, max_tokens=max_tokens, detokenize=False, ignore_eos=True)
        outs = llm.generate(PROMPTS, sp)
        return [list(o.outputs[0].token_ids) for o in outs]
    finally:
        llm.shutdown()


@pytest.mark.parametrize("arch,ep", [("Qwen3ForCausalLM", False), ("Qwen3MoeForCausalLM", False),
                                     ("Qwen3MoeForCausalLM", True)])
def test_two_rank_engine_matches_single_rank_cpu(arch, ep):
    import torch.distributed as dist
    one = _run(arch, 1)
    try:
        two = _run(arch, 2, ep)
    finally:
        if dist.is_initialized():
            from vllm_omni_b200.parallel import parallel_state as ps
            ps.destroy_model_parallel()
            ps.destroy_distributed_environment()
    assert two == one
    assert all(len(t) == 8 for t in two)


def test_decoder_shards_sum_to_the_full_model():
    """Shard arithmetic without processes: the two ranks' partial products of every row-parallel layer
    add up to the unsharded layer (KV heads replicated when there are fewer of them than ranks)."""
    from vllm_omni_b200.models.qwen_decoder import DecoderConfig, QwenDecoderModel

    class FakeGroup:
        def __init__(self, r, w):
            self.rank_in_group, self.world_size = r, w

        def all_reduce(self, x):
            return x
    cfg = DecoderConfig(vocab_size=64, hidden_size=64, num_hidden_layers=1, num_attention_heads=4,
                        num_key_value_heads=1, head_dim=16, intermediate_size=96)
    torch.manual_seed(0)
    full = QwenDecoderModel(cfg, dtype=torch.float32, device="cpu")
    parts = []
    for r in range(2):
        torch.manual_seed(0)
        m = QwenDecoderModel(cfg, dtype=torch.float32, device="cpu")
        m.enable_tensor_parallel(FakeGroup(r, 2), mode="nccl")
        assert m.local_heads == (2, 1)
        parts.append(m)
    x = torch.randn(5, 64)
    lf = full.layers[0]
    qkv_full = lf.qkv_proj(x)
    o_full = lf.o_proj(qkv_full[:, :64])
    o_sum = sum(p.layers[0].o_proj(p.layers[0].qkv_proj(x)[:, :32]) for p in parts)
    assert torch.allclose(o_sum, o_full, atol=1e-5)
    import torch.nn.functional as F
    h_full = lf.gate_up(x)
    d_full = lf.down(F.silu(h_full[:, :96]) * h_full[:, 96:])
    d_sum = 0
    for p in parts:
        h = p.layers[0].gate_up(x)
        d_sum = d_sum + p.layers[0].down(F.silu(h[:, :48]) * h[:, 48:])
    assert torch.allclose(d_sum, d_full, atol=1e-5)


@pytest.mark.gpu
def test_two_gpu_engine_matches_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.distributed as dist
    ov = {"tiny": True, "head_dim": 128, "vocab_size": 600}
    one = _run("Qwen3MoeForCausalLM", 1, device=None, overrides=ov)
    try:
        two = _run("Qwen3MoeForCausalLM", 2, True, device=None, overrides=ov)
    finally:
        if dist.is_initialized():
            from vllm_omni_b200.parallel import parallel_state as ps
            ps.destroy_model_parallel()
            ps.destroy_distributed_environment()
    # bf16 partial sums are added in another order: allow a late divergence, not an early one
    agree = sum(a[:4] == b[:4] for a, b in zip(one, two))
    assert agree == len(one), (one, two)
