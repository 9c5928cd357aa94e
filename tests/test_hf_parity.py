"""Checkpoint compatibility of the decoder: a random-weight Hugging Face model's ``state_dict`` is
loaded by HF parameter names and the logits agree (fp32, CPU).  Covers the dense Qwen2 layout
(q/k/v biases, no q/k norm), Qwen3 (per-head q/k RMSNorm) and Qwen3-MoE (stacked experts)."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from vllm_omni_b200.models.qwen_decoder import DecoderConfig, ModelBatch, PrefillSeg, QwenDecoderModel

BASE = dict(vocab_size=128, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
            intermediate_size=96, max_position_embeddings=512)


def _compare(hf, extra):
    d = hf.config.to_dict()
    d.update(extra)
    cfg = DecoderConfig.from_dict(d)
    m = QwenDecoderModel(cfg, torch.float32, "cpu")
    sd = hf.state_dict()
    loaded = m.load_weights(sd.items())
    assert loaded == set(sd), set(sd) - loaded
    T = 19
    ids = torch.randint(0, cfg.vocab_size, (T,))
    with torch.no_grad():
        ref = hf(ids[None]).logits[0]
        b = ModelBatch(ids, torch.arange(T), torch.full((T,), -1, dtype=torch.int32), [PrefillSeg(0, T, 0, None)])
        h, _ = m(b, None)
        out = m.compute_logits(h)
    assert (out - ref).abs().max().item() < 1e-4 * max(1.0, ref.abs().max().item())


def test_qwen2_dense_with_bias():
    torch.manual_seed(0)
    hf = transformers.Qwen2ForCausalLM(transformers.Qwen2Config(**BASE)).float().eval()
    _compare(hf, dict(qk_norm=False, attention_bias=True))


def test_qwen3_dense_qk_norm():
    torch.manual_seed(1)
    hf = transformers.Qwen3ForCausalLM(transformers.Qwen3Config(**BASE, head_dim=32)).float().eval()
    _compare(hf, {})


def test_qwen3_moe_stacked_experts():
    torch.manual_seed(2)
    c = transformers.Qwen3MoeConfig(**BASE, head_dim=32, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=48,
                                    decoder_sparse_step=1, mlp_only_layers=[], norm_topk_prob=True)
    hf = transformers.Qwen3MoeForCausalLM(c).float().eval()
    _compare(hf, {})


def test_per_expert_checkpoint_names():
    """Checkpoints on disk name every expert separately (``mlp.experts.N.gate_proj.weight``)."""
    torch.manual_seed(3)
    c = transformers.Qwen3MoeConfig(**BASE, head_dim=32, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=48,
                                    decoder_sparse_step=1, mlp_only_layers=[], norm_topk_prob=True)
    hf = transformers.Qwen3MoeForCausalLM(c).float().eval()
    cfg = DecoderConfig.from_dict(c.to_dict())
    flat = {}
    for k, v in hf.state_dict().items():
        if k.endswith("mlp.experts.gate_up_proj"):
            for e in range(4):
                flat[k.replace("gate_up_proj", f"{e}.gate_proj.weight")] = v[e, :48]
                flat[k.replace("gate_up_proj", f"{e}.up_proj.weight")] = v[e, 48:]
        elif k.endswith("mlp.experts.down_proj"):
            for e in range(4):
                flat[k.replace("down_proj", f"{e}.down_proj.weight")] = v[e]
        else:
            flat[k] = v
    a, b = QwenDecoderModel(cfg, torch.float32, "cpu"), QwenDecoderModel(cfg, torch.float32, "cpu")
    a.load_weights(hf.state_dict().items())
    assert b.load_weights(flat.items()) == set(flat)
    for (n, p), (_, q) in zip(a.named_parameters(), b.named_parameters()):
        assert torch.equal(p, q), n
