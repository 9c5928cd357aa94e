"""Qwen2.5-Omni-style pipeline (thinker -> talker -> token2wav) on CPU with the tiny geometry:
the thinker hands its last-layer hidden states to the talker, the talker's codec tokens go
through the flow-matching DiT (Runge-Kutta solver, guidance) and the vocoder."""
import math
import textwrap

import pytest
import torch

from vllm_omni_b200.entrypoints.omni import Omni

YAML = textwrap.dedent("""
    async_chunk: false
    stage_args:
      - stage_id: 0
        stage_type: llm
        runtime: {devices: "0", max_batch_size: 4}
        engine_args: {model_stage: thinker, model_arch: Qwen2_5OmniForConditionalGeneration, worker_type: ar,
                      engine_output_type: latent, device: cpu, num_gpu_blocks: 64, max_num_batched_tokens: 64,
                      model_overrides: {tiny: true}}
        final_output: true
        final_output_type: text
        default_sampling_params: {temperature: 0.0, max_tokens: 4}
      - stage_id: 1
        stage_type: llm
        runtime: {devices: "0", max_batch_size: 4}
        engine_args: {model_stage: talker, model_arch: Qwen2_5OmniForConditionalGeneration, worker_type: ar,
                      engine_output_type: latent, device: cpu, num_gpu_blocks: 64, model_overrides: {tiny: true}}
        engine_input_source: [0]
        custom_process_input_func: vllm_omni.model_executor.stage_input_processors.qwen2_5_omni.thinker2talker
        default_sampling_params: {temperature: 0.0, max_tokens: 6, detokenize: false, stop_token_ids: [94]}
      - stage_id: 2
        stage_type: llm
        runtime: {devices: "0", max_batch_size: 4}
        engine_args: {model_stage: code2wav, model_arch: Qwen2_5OmniForConditionalGeneration,
                      worker_type: generation, engine_output_type: audio, device: cpu, model_overrides: {tiny: true}}
        engine_input_source: [1]
        custom_process_input_func: vllm_omni_b200.models.stage_input_processors.qwen2_5_omni.talker2code2wav
        final_output: true
        final_output_type: audio
    """)


@pytest.fixture(scope="module")
def omni(tmp_path_factory):
    p = tmp_path_factory.mktemp("cfg") / "tiny_qwen2_5_omni.yaml"
    p.write_text(YAML)
    o = Omni("qwen2.5-omni-tiny", stage_configs_path=str(p))
    yield o
    o.close()


def test_three_stage_text_and_audio(omni):
    mel = torch.randn(16, 40, generator=torch.Generator().manual_seed(0))
    prompt = {"prompt_token_ids": [506, 10, 11, 500, 12, 507, 506, 13], "multi_modal_data": {"audio": [mel]}}
    sps = [s.default_sampling_params() for s in omni.stage_list]
    outs = omni.generate([prompt], sps)
    by_type = {o.final_output_type: o for o in outs}
    assert len(by_type["text"].outputs[0].token_ids) == 4
    wav = by_type["audio"].multimodal_output["audio"]
    # up to 6 codec tokens x 2 mel frames x up-sampling 4
    assert wav.dim() == 1 and wav.numel() % 8 == 0 and 8 <= wav.numel() <= 6 * 8
    assert torch.isfinite(wav).all() and wav.abs().max() <= 1.0


def test_rk4_and_time_grid():
    from vllm_omni_b200.models.qwen2_5_omni.token2wav import rk4_38_integrate, sway_time_grid
    x = rk4_38_integrate(lambda t, x: x, torch.ones(1, dtype=torch.float64), torch.linspace(0, 1, 11, dtype=torch.float64))
    assert abs(float(x) - math.e) < 1e-5
    t = sway_time_grid(10, -1.0, "cpu")
    assert t[0] == 0 and abs(float(t[-1]) - 1.0) < 1e-6 and bool((t[1:] > t[:-1]).all())
    # sway -1 spends more steps early: the warped grid lies below the uniform one
    assert bool((t[1:-1] < torch.linspace(0, 1, 10)[1:-1]).all())


def test_dit_block_locality():
    """Every layer sees its own block of frames; the listed layers also the previous / next block."""
    from vllm_omni_b200.models.qwen2_5_omni.config import Qwen25OmniConfig
    from vllm_omni_b200.models.qwen2_5_omni.token2wav import Token2WavDiT
    c = Qwen25OmniConfig.tiny().dit
    m = Token2WavDiT(c)
    d = m.block_diff(40, "cpu")
    bs = c.block_size
    assert int(d[0, bs - 1]) == 0 and int(d[0, bs]) == 1 and int(d[2 * bs, 0]) == -2
    assert [(l.look_ahead, l.look_backward) for l in m.transformer_blocks] == [(0, 1), (1, 0), (0, 1)]
    # a change in block 3 reaches block 0 through at most the backward-looking layers: not at all here
    torch.manual_seed(0)
    for p in m.parameters():
        if p.dim() > 1:
            torch.nn.init.normal_(p, 0, 0.2)
    x, ref, xv = torch.randn(1, 40, c.mel_dim), torch.randn(1, 9, c.mel_dim), torch.randn(1, 40, c.enc_emb_dim)
    codes = torch.randint(1, 90, (1, 20))
    y0 = m(x, ref, xv, codes, torch.tensor(0.3), apply_cfg=False)
    x2 = x.clone()
    x2[:, 3 * bs:] += 1.0
    y1 = m(x2, ref, xv, codes, torch.tensor(0.3), apply_cfg=False)
    assert torch.allclose(y0[:, :bs], y1[:, :bs], atol=1e-6) and not torch.allclose(y0[:, 3 * bs:], y1[:, 3 * bs:])
