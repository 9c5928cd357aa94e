"""Three-stage Qwen3-Omni-style pipeline (thinker -> talker -> code2wav) on CPU with the tiny
geometry: text + audio features in, text tokens and a waveform out, through the Omni API and a
stage-config YAML."""
import textwrap

import pytest
import torch

from vllm_omni_b200.entrypoints.omni import Omni
from vllm_omni_b200.inputs import SamplingParams

YAML = textwrap.dedent("""
    async_chunk: false
    stage_args:
      - stage_id: 0
        stage_type: llm
        runtime: {devices: "0", max_batch_size: 4}
        engine_args: {model_stage: thinker, model_arch: Qwen3OmniMoeForConditionalGeneration, worker_type: ar,
                      engine_output_type: latent, device: cpu, num_gpu_blocks: 64, max_num_batched_tokens: 64,
                      model_overrides: {tiny: true}}
        final_output: true
        final_output_type: text
        default_sampling_params: {temperature: 0.0, max_tokens: 5}
      - stage_id: 1
        stage_type: llm
        runtime: {devices: "0", max_batch_size: 4}
        engine_args: {model_stage: talker, model_arch: Qwen3OmniMoeForConditionalGeneration, worker_type: ar,
                      engine_output_type: latent, device: cpu, num_gpu_blocks: 64, model_overrides: {tiny: true}}
        engine_input_source: [0]
        custom_process_input_func: vllm_omni.model_executor.stage_input_processors.qwen3_omni.thinker2talker
        default_sampling_params: {temperature: 0.0, max_tokens: 7, detokenize: false, stop_token_ids: [66]}
      - stage_id: 2
        stage_type: llm
        runtime: {devices: "0", max_batch_size: 4}
        engine_args: {model_stage: code2wav, model_arch: Qwen3OmniMoeForConditionalGeneration,
                      worker_type: generation, engine_output_type: audio, device: cpu, model_overrides: {tiny: true}}
        engine_input_source: [1]
        custom_process_input_func: vllm_omni_b200.models.stage_input_processors.qwen3_omni.talker2code2wav
        final_output: true
        final_output_type: audio
    """)


@pytest.fixture(scope="module")
def omni(tmp_path_factory):
    p = tmp_path_factory.mktemp("cfg") / "tiny_qwen3_omni.yaml"
    p.write_text(YAML)
    o = Omni("qwen3-omni-tiny", stage_configs_path=str(p))
    yield o
    o.close()


def _prompt(n_audio_frames=40):
    mel = torch.randn(16, n_audio_frames, generator=torch.Generator().manual_seed(0))
    ids = [506, 509, 11, 500, 12, 507, 506, 510, 13]    # user turn with one audio placeholder, assistant header
    return {"prompt_token_ids": ids, "multi_modal_data": {"audio": [mel]}}


def test_three_stage_text_and_audio(omni):
    sps = [s.default_sampling_params() for s in omni.stage_list]
    sps[1].stop_token_ids, sps[1].ignore_eos = [], True     # random weights may pick the stop code first: speak all 7 frames
    outs = omni.generate([_prompt(), _prompt(24)], sps)
    by_type = {}
    for o in outs:
        by_type.setdefault(o.final_output_type, []).append(o)
    assert len(by_type["text"]) == 2 and len(by_type["audio"]) == 2
    t = by_type["text"][0]
    assert t.stage_id == 0 and len(t.outputs[0].token_ids) == 5
    a = by_type["audio"][0]
    wav = a.multimodal_output["audio"]
    # 7 codec frames (or fewer if the stop code came up) x total up-sampling 16
    assert wav.dim() == 1 and 1 <= wav.numel() <= 7 * 16   # the decoder trims a few samples per transposed conv
    assert torch.isfinite(wav).all() and wav.abs().max() <= 1.0
    s = omni.metrics.build_summary()
    assert s["overall"]["e2e_requests"] >= 2 and len(s["stages"]) >= 6


def test_thinker_expands_audio_placeholder(omni):
    from vllm_omni_b200.entrypoints.stage_runtime import inproc_adapter
    llm = inproc_adapter(0).llm
    req = llm.add_request("probe", _prompt(40), SamplingParams(temperature=0.0, max_tokens=1))
    n_audio = llm.model.audio_tower.output_length(40)
    assert req.num_prompt_tokens == 8 + n_audio
    assert req.prompt_embeds.shape == (8 + n_audio, 64)
    pos = req.runtime_state["mrope_positions"]
    assert pos.shape == (3, 8 + n_audio) and int(pos[0, -1]) == 8 + n_audio - 1
    llm.abort_request(["probe"])


def test_thinker_image_deepstack_reaches_the_decoder(omni):
    """An image placeholder expands to the merged patch count; the vision tower's deep-stack features
    are added after the first decoder layer(s) on exactly the image rows, also when the prompt is
    prefilled in two chunks."""
    from types import SimpleNamespace
    from vllm_omni_b200.entrypoints.stage_runtime import inproc_adapter
    from vllm_omni_b200.models.qwen_decoder import ModelBatch, PrefillSeg
    llm = inproc_adapter(0).llm
    th = llm.model
    img = torch.randn(3, 16, 16, generator=torch.Generator().manual_seed(1))     # 4x4 patches -> 2x2 merged tokens
    ids = [506, 10, 501, 11, 507]
    req = llm.add_request("img", {"prompt_token_ids": ids, "multi_modal_data": {"image": [img]}},
                          SamplingParams(temperature=0.0, max_tokens=1))
    try:
        assert req.num_prompt_tokens == 4 + 4
        rows, vals = req.runtime_state["deepstack"]
        assert rows.tolist() == [2, 3, 4, 5] and len(vals) == 1 and vals[0].shape == (4, 64)
        T = req.num_prompt_tokens
        pos = req.runtime_state["mrope_positions"]

        def run(chunks):
            outs, start = [], 0
            for n in chunks:
                b = ModelBatch(torch.tensor(req.prompt_token_ids[start:start + n]), pos[:, start:start + n],
                               torch.full((n,), -1, dtype=torch.int32), [PrefillSeg(0, n, 0, None)],
                               input_embeds=req.prompt_embeds[start:start + n],
                               embeds_mask=torch.ones(n, dtype=torch.bool))
                sched = SimpleNamespace(scheduled=[SimpleNamespace(request=req, start=start, num_new_tokens=n, is_prefill=True)])
                outs.append(th._deepstack(b, sched))
                start += n
            return outs
        whole = run([T])[0][0]
        assert torch.equal(whole[2:6], vals[0]) and whole[:2].abs().sum() == 0 and whole[6:].abs().sum() == 0
        a, b = run([3, T - 3])
        assert torch.equal(torch.cat([a[0], b[0]]), whole)
        # the features change the hidden states of the image rows (and, through attention, later rows)
        b0 = ModelBatch(torch.tensor(req.prompt_token_ids), pos, torch.full((T,), -1, dtype=torch.int32),
                        [PrefillSeg(0, T, 0, None)], input_embeds=req.prompt_embeds, embeds_mask=torch.ones(T, dtype=torch.bool))
        h0, _ = th.decoder(b0, None)
        h1, _ = th.decoder(b0, None, deepstack=[whole])
        assert torch.equal(h0[:2], h1[:2]) and (h0[2:] - h1[2:]).abs().max() > 0
    finally:
        llm.abort_request(["img"])


def test_talker_prompt_follows_chatml_turns():
    """System turn dropped, user turn row per token (audio row from the hidden states), assistant turn
    = 3 header rows + 4 x pad + bos + first reply token with the codec control tokens added on the
    last six rows; the other reply tokens and tts-eos wait for the decode steps."""
    from types import SimpleNamespace
    from vllm_omni_b200.models.qwen3_omni.config import Qwen3OmniConfig
    from vllm_omni_b200.models.qwen3_omni.talker import Qwen3OmniMoeTalker
    torch.manual_seed(0)
    cfg = Qwen3OmniConfig.tiny()
    tk = Qwen3OmniMoeTalker(cfg, torch.float32, "cpu")
    prompt = [506, 508, 20, 507, 506, 509, 21, 500, 22, 507, 506, 510, 30]
    gen = [40, 41, 42]
    L = len(prompt) + len(gen)
    emb, hid = torch.randn(L, 64), torch.randn(L, 64)
    e3 = {k: torch.randn(1, 64) for k in ("tts_bos_embed", "tts_eos_embed", "tts_pad_embed")}
    req = SimpleNamespace(additional_information=dict(thinker_embeddings=emb, thinker_hidden_states=hid,
                                                      thinker_sequences=prompt + gen, thinker_input_ids=prompt,
                                                      voice_type="Chelsie", **e3),
                          runtime_state={}, prompt_embeds=None, prompt_token_ids=None)
    tk.preprocess_request(req)
    head = req.prompt_embeds
    tp, hp, codec = tk.text_projection, tk.hidden_projection, tk.decoder.embed_tokens
    pad, bos, eos = tp(e3["tts_pad_embed"]), tp(e3["tts_bos_embed"]), tp(e3["tts_eos_embed"])
    assert head.shape == (6 + 9, 48) and len(req.prompt_token_ids) == 15
    user = tp(emb[4:10])
    user[3] = hp(hid[7:8])[0]
    assert torch.allclose(head[:6], user, atol=1e-6)
    a = head[6:]
    assert torch.allclose(a[:3], tp(emb[10:13]), atol=1e-6)
    ctrl = [cfg.codec_nothink_id, cfg.codec_think_bos_id, cfg.codec_think_eos_id, cfg.speaker_ids["chelsie"]]
    for i, c in enumerate(ctrl):
        assert torch.allclose(a[3 + i], pad[0] + codec[c], atol=1e-6)
    assert torch.allclose(a[7], bos[0] + codec[cfg.codec_pad_id], atol=1e-6)
    assert torch.allclose(a[8], tp(emb[13:14])[0] + codec[cfg.codec_bos_id], atol=1e-6)
    trailing = req.runtime_state["text_steps"]
    assert torch.allclose(trailing, torch.cat([tp(emb[14:16]), eos]), atol=1e-6)
    assert tk.speaker_token("nobody") == cfg.speaker_ids["ethan"]        # unknown voice -> the first listed voice


def test_every_stage_in_its_own_process_matches_the_in_process_pipeline(omni, tmp_path):
    """``runtime.process: true`` on all three stages: payloads cross the edges through shared-memory
    connectors, and text tokens and waveform equal the single-process run."""
    y = tmp_path / "procs.yaml"
    y.write_text(YAML.replace("max_batch_size: 4}", "max_batch_size: 4, process: true}"))
    sps = [s.default_sampling_params() for s in omni.stage_list]
    sps[1].stop_token_ids, sps[1].ignore_eos = [], True
    ref = omni.generate([_prompt(40)], sps)
    o = Omni("qwen3-omni-tiny", stage_configs_path=str(y))
    try:
        assert all(not s.in_process for s in o.stage_list)
        out = o.generate([_prompt(40)], sps)
    finally:
        o.close()
    pick = lambda outs, kind: [x for x in outs if x.final_output_type == kind][0]
    assert list(pick(out, "text").request_output.outputs[0].token_ids) == list(pick(ref, "text").request_output.outputs[0].token_ids)
    a, b = pick(out, "audio").multimodal_output["audio"], pick(ref, "audio").multimodal_output["audio"]
    assert a.shape == b.shape and torch.allclose(a, b, atol=1e-6)
