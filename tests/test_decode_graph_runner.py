"""Static-buffer decode step (the body a CUDA graph replays): bucket padding, slot masking and
MRoPE positions give the same hidden states and cache contents as the direct decoder call."""
import pytest
import torch

from vllm_omni_b200.engine.graph_runner import DecodeGraphRunner
from vllm_omni_b200.models.qwen_decoder import DecoderConfig, ModelBatch, PrefillSeg, QwenDecoderModel


def _setup(mrope):
    torch.manual_seed(0)
    cfg = DecoderConfig(vocab_size=64, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                        head_dim=8, intermediate_size=48, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=16,
                        mrope_section=(2, 1, 1) if mrope else None, mrope_interleaved=mrope)
    m = QwenDecoderModel(cfg, torch.float32, "cpu")
    nb, bs = 16, 4
    mk = lambda: [(torch.zeros(nb, bs, 2, 8), torch.zeros(nb, bs, 2, 8)) for _ in range(2)]
    return cfg, m, mk, bs


def _prefill(m, caches, tables, lens, bs):
    for i, L in enumerate(lens):
        ids = torch.arange(L) + 3 * i
        slots = torch.tensor([tables[i][t // bs] * bs + t % bs for t in range(L)], dtype=torch.int32)
        pos = torch.arange(L)
        if m.cfg.mrope_section is not None:
            pos = pos[None].expand(3, -1)
        m(ModelBatch(ids, pos, slots, [PrefillSeg(0, L, 0, torch.tensor(tables[i], dtype=torch.int32))]), caches)


def _decode_batch(cfg, tables, lens, bs, with_embeds):
    n = len(lens)
    ids = torch.tensor([7, 9, 11][:n])
    pos = torch.tensor(lens)
    if cfg.mrope_section is not None:
        pos = torch.stack([pos, pos + 1, pos + 2])
    slots = torch.tensor([tables[i][lens[i] // bs] * bs + lens[i] % bs for i in range(n)], dtype=torch.int32)
    w = max(len(t) for t in tables)
    bt = torch.tensor([t + [0] * (w - len(t)) for t in tables], dtype=torch.int32)
    kw = {}
    if with_embeds:
        g = torch.Generator().manual_seed(1)
        kw = dict(input_embeds=torch.randn(n, cfg.hidden_size, generator=g), embeds_mask=torch.tensor([True, False, True][:n]))
    return ModelBatch(ids, pos, slots, [], decode_rows=torch.arange(n), decode_block_tables=bt,
                      decode_seq_lens=torch.tensor([L + 1 for L in lens], dtype=torch.int32), **kw)


def _check(mrope, with_embeds):
    cfg, m, mk, bs = _setup(mrope)
    tables, lens = [[0, 1, 2], [3, 4], [5, 6, 7]], [9, 5, 10]
    ca, cb = mk(), mk()
    _prefill(m, ca, tables, lens, bs)
    _prefill(m, cb, tables, lens, bs)
    batch = _decode_batch(cfg, tables, lens, bs, with_embeds)
    ref, cap_ref = m(batch, ca, capture_layers=(0, 1))
    r = DecodeGraphRunner(m, cb, max_blocks=4, capture_layers=(0, 1), buckets=(1, 4, 8))
    assert r.supports(batch) and not r.use_graph
    out, cap = r.run(batch)
    assert out.shape == ref.shape and torch.allclose(out, ref, atol=1e-5)
    assert all(torch.allclose(cap[k], cap_ref[k], atol=1e-5) for k in cap_ref)
    for (ka, va), (kb, vb) in zip(ca, cb):           # padding rows wrote nothing
        assert torch.equal(ka, kb) and torch.equal(va, vb)
    # a second step of another size reuses / creates buckets and still matches
    b2 = _decode_batch(cfg, tables[:1], lens[:1], bs, with_embeds)
    ref2, _ = m(b2, ca)
    out2, _ = r.run(b2)
    assert torch.allclose(out2, ref2, atol=1e-5) and sorted(r._state) == [1, 4] and r.replays == 2


def test_plain_positions():
    _check(mrope=False, with_embeds=False)


def test_mrope_positions_and_embedding_overlay():
    _check(mrope=True, with_embeds=True)


def test_batches_with_prefill_segments_or_wide_tables_are_refused():
    cfg, m, mk, bs = _setup(False)
    r = DecodeGraphRunner(m, mk(), max_blocks=2, buckets=(1, 2))
    tables, lens = [[0, 1, 2]], [9]
    assert not r.supports(_decode_batch(cfg, tables, lens, bs, False))            # table wider than the static buffer
    b = ModelBatch(torch.arange(3), torch.arange(3), torch.zeros(3, dtype=torch.int32), [PrefillSeg(0, 3, 0, None)])
    assert not r.supports(b)
    three = _decode_batch(cfg, [[0], [1], [2]], [1, 1, 1], bs, False)
    assert not r.supports(three)                                                    # more rows than the largest bucket


def test_engine_with_the_static_buffer_step_generates_the_same_tokens(monkeypatch):
    """The AR engine with the runner switched on (eager static-buffer steps on CPU) samples the same
    greedy tokens as the plain engine."""
    from vllm_omni_b200.entrypoints.omni_llm import OmniLLM
    from vllm_omni_b200.inputs import SamplingParams
    kw = dict(model_arch="Qwen3OmniMoeForConditionalGeneration", model_stage="thinker", device="cpu", num_gpu_blocks=64,
              model_overrides={"tiny": True}, engine_output_type="latent")
    prompts = [{"prompt_token_ids": [506, 509, 11, 12, 507, 506, 510, 13]}, {"prompt_token_ids": [506, 509, 20, 507, 506, 510]}]
    sp = SamplingParams(temperature=0.0, max_tokens=6, detokenize=False)

    def run():
        llm = OmniLLM(None, **kw)
        outs = llm.generate(prompts, sp)
        return llm, [list(o.outputs[0].token_ids) for o in outs]
    _, plain = run()
    monkeypatch.setenv("OMNI_AR_CUDA_GRAPH", "1")
    llm, graphed = run()
    r = llm.engine.runner.graph_runner if hasattr(llm.engine, "runner") else None
    assert graphed == plain
    assert r is not None and r.replays > 0


@pytest.mark.gpu
def test_captured_decode_graph_generates_the_same_tokens_on_gpu(monkeypatch):
    """On a GPU the decode step is replayed from a CUDA graph by default; greedy tokens equal the eager
    engine's (two requests fill the two-row bucket, so both runs launch identical kernels)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from vllm_omni_b200.entrypoints.omni_llm import OmniLLM
    from vllm_omni_b200.inputs import SamplingParams
    kw = dict(model_arch="Qwen3MoeForCausalLM", device="cuda", num_gpu_blocks=64, block_size=16,
              model_overrides={"tiny": True, "head_dim": 128, "vocab_size": 600, "moe": True})
    prompts = [{"prompt_token_ids": [3, 17, 42, 99, 7, 150, 23, 8, 64]}, {"prompt_token_ids": [5, 9, 11, 300, 2, 77]}]
    sp = SamplingParams(temperature=0.0, max_tokens=12, detokenize=False, ignore_eos=True)

    def run(flag):
        monkeypatch.setenv("OMNI_AR_CUDA_GRAPH", flag)
        llm = OmniLLM(None, **kw)
        outs = llm.generate(prompts, sp)
        return llm, [list(o.outputs[0].token_ids) for o in outs]
    _, eager = run("0")
    monkeypatch.delenv("OMNI_AR_CUDA_GRAPH")
    llm, graphed = run("1")
    r = llm.engine.runner.graph_runner
    assert r is not None and r.use_graph and r.replays > 0 and any(b.graph is not None for b in r._state.values())
    assert graphed == eager
