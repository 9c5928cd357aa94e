"""Qwen3-TTS as a single generation stage on CPU (tiny geometry), and the private decode session
it runs on: incremental steps over the paged cache equal one full causal forward."""
import textwrap

import torch

from vllm_omni_b200.entrypoints.omni import Omni
from vllm_omni_b200.inputs import SamplingParams

YAML = textwrap.dedent("""
    stage_args:
      - stage_id: 0
        stage_type: llm
        runtime: {devices: "0", max_batch_size: 2}
        engine_args: {model_stage: qwen3_tts, model_arch: Qwen3TTSForConditionalGeneration, worker_type: generation,
                      engine_output_type: audio, device: cpu, model_overrides: {tiny: true}}
        final_output: true
        final_output_type: audio
        default_sampling_params: {temperature: 0.0, max_tokens: 8, seed: 1}
    """)


def test_tts_stage_produces_waveform(tmp_path):
    p = tmp_path / "tiny_tts.yaml"
    p.write_text(YAML)
    omni = Omni("qwen3-tts-tiny", stage_configs_path=str(p))
    try:
        prompt = {"prompt_token_ids": [11, 12, 13, 14, 15], "additional_information": {"speaker": 1, "language": 1}}
        outs = omni.generate([prompt], [SamplingParams(temperature=0.0, max_tokens=8, seed=1)])
        assert len(outs) == 1 and outs[0].final_output_type == "audio"
        wav = outs[0].multimodal_output["audio"]
        assert wav.dim() == 1 and 0 < wav.numel() <= 8 * 16
        assert torch.isfinite(wav).all() and wav.abs().max() <= 1.0
    finally:
        omni.close()


def test_local_decode_session_matches_full_forward():
    from vllm_omni_b200.models.local_decode import LocalDecodeSession
    from vllm_omni_b200.models.qwen_decoder import DecoderConfig, QwenDecoderModel, reference_forward
    cfg = DecoderConfig(vocab_size=128, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, head_dim=16, intermediate_size=96)
    torch.manual_seed(0)
    m = QwenDecoderModel(cfg, torch.float32, "cpu")
    ids = torch.randint(0, 128, (23,))
    ref = reference_forward(m, ids)
    s = LocalDecodeSession(m, 40)
    got = [s.prefill(ids=ids[:9])]
    for t in range(9, 23):
        got.append(s.step(token=int(ids[t])))
    assert torch.allclose(torch.cat(got, 0), ref, atol=2e-4, rtol=1e-3)
    s.reset()
    again = s.prefill(ids=ids[:9])
    assert torch.allclose(again, ref[:9], atol=2e-4, rtol=1e-3)
