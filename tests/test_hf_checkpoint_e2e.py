"""A Hugging Face Qwen3-Omni checkpoint on disk (``save_pretrained``: config.json + safetensors
with per-expert weight names) served by the three-stage pipeline through ``Omni``: every stage
finds its own tensors, greedy thinker tokens equal those of ``transformers``' ``generate`` and the
talker + code2wav stages deliver a waveform."""
import textwrap

import pytest
import torch

transformers = pytest.importorskip("transformers")

from vllm_omni_b200.entrypoints.omni import Omni

ROPE = dict(rope_theta=1e6, rope_type="default", mrope_section=[4, 2, 2], mrope_interleaved=True)
THINKER = dict(
    audio_config=dict(num_mel_bins=16, d_model=32, encoder_layers=1, encoder_attention_heads=2, encoder_ffn_dim=64,
                      downsample_hidden_size=8, output_dim=64, n_window=8, n_window_infer=32, max_source_positions=64),
    vision_config=dict(depth=2, hidden_size=32, num_heads=2, intermediate_size=64, patch_size=4, temporal_patch_size=2,
                       spatial_merge_size=2, out_hidden_size=64, num_position_embeddings=16, deepstack_visual_indexes=[0]),
    text_config=dict(vocab_size=512, hidden_size=64, intermediate_size=96, num_hidden_layers=3, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=16, moe_intermediate_size=32, num_experts=4, num_experts_per_tok=2,
                     norm_topk_prob=True, max_position_embeddings=512, rope_parameters=ROPE),
    audio_token_id=500, image_token_id=501, video_token_id=502)
TALKER = dict(
    text_config=dict(vocab_size=96, hidden_size=48, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=16, moe_intermediate_size=32, shared_expert_intermediate_size=24,
                     num_experts=4, num_experts_per_tok=2, norm_topk_prob=True, max_position_embeddings=512,
                     rope_parameters=ROPE),
    code_predictor_config=dict(vocab_size=64, hidden_size=48, intermediate_size=64, num_hidden_layers=1,
                               num_attention_heads=4, num_key_value_heads=2, head_dim=16, num_code_groups=4,
                               max_position_embeddings=64),
    thinker_hidden_size=64, num_code_groups=4, accept_hidden_layer=2, spatial_merge_size=2, codec_eos_token_id=66,
    codec_bos_id=65, codec_pad_id=64, codec_nothink_id=67, audio_token_id=500, image_token_id=501, video_token_id=502)
C2W = dict(codebook_size=64, hidden_size=32, num_attention_heads=2, num_key_value_heads=2, sliding_window=5,
           intermediate_size=64, num_hidden_layers=1, num_quantizers=4, upsample_rates=[4, 2], upsampling_ratios=[2],
           decoder_dim=32, max_position_embeddings=512)

YAML = textwrap.dedent("""
    async_chunk: false
    stage_args:
      - stage_id: 0
        stage_type: llm
        runtime: {devices: "0", max_batch_size: 4}
        engine_args: {model_stage: thinker, model_arch: Qwen3OmniMoeForConditionalGeneration, worker_type: ar,
                      engine_output_type: latent, device: cpu, dtype: float32, num_gpu_blocks: 64,
                      max_num_batched_tokens: 64}
        final_output: true
        final_output_type: text
        default_sampling_params: {temperature: 0.0, max_tokens: 6, detokenize: false}
      - stage_id: 1
        stage_type: llm
        runtime: {devices: "0", max_batch_size: 4}
        engine_args: {model_stage: talker, model_arch: Qwen3OmniMoeForConditionalGeneration, worker_type: ar,
                      engine_output_type: latent, device: cpu, dtype: float32, num_gpu_blocks: 64}
        engine_input_source: [0]
        custom_process_input_func: vllm_omni_b200.models.stage_input_processors.qwen3_omni.thinker2talker
        default_sampling_params: {temperature: 0.0, max_tokens: 7, detokenize: false, stop_token_ids: [66]}
      - stage_id: 2
        stage_type: llm
        runtime: {devices: "0", max_batch_size: 4}
        engine_args: {model_stage: code2wav, model_arch: Qwen3OmniMoeForConditionalGeneration,
                      worker_type: generation, engine_output_type: audio, device: cpu, dtype: float32}
        engine_input_source: [1]
        custom_process_input_func: vllm_omni_b200.models.stage_input_processors.qwen3_omni.talker2code2wav
        final_output: true
        final_output_type: audio
    """)


@pytest.fixture(scope="module")
def checkpoint(tmp_path_factory):
    from transformers.models.qwen3_omni_moe import modeling_qwen3_omni_moe as M
    from transformers.models.qwen3_omni_moe.configuration_qwen3_omni_moe import Qwen3OmniMoeConfig
    torch.manual_seed(0)
    cfg = Qwen3OmniMoeConfig(thinker_config=THINKER, talker_config=TALKER, code2wav_config=C2W, enable_audio_output=True,
                             tts_bos_token_id=503, tts_eos_token_id=504, tts_pad_token_id=505, im_start_token_id=506,
                             im_end_token_id=507)
    hf = M.Qwen3OmniMoeForConditionalGeneration(cfg)
    for _, p in hf.named_parameters():
        if p.dim() > 1:
            torch.nn.init.normal_(p, 0, 0.05)
    hf = hf.float().eval()
    d = tmp_path_factory.mktemp("qwen3_omni_hf")
    hf.save_pretrained(str(d))
    (d / "stages.yaml").write_text(YAML)
    return hf, d


def test_pipeline_serves_hf_checkpoint(checkpoint):
    hf, d = checkpoint
    from vllm_omni_b200.entrypoints.stage_runtime import inproc_adapter
    ids = [506, 10, 11, 12, 507, 506, 13]
    o = Omni(str(d), stage_configs_path=str(d / "stages.yaml"))
    try:
        outs = o.generate([{"prompt_token_ids": ids}])
        text = [x for x in outs if x.final_output_type == "text"][0]
        audio = [x for x in outs if x.final_output_type == "audio"][0]
        mine = list(text.request_output.outputs[0].token_ids)
        assert audio.multimodal_output["audio"].numel() > 0
        # every stage took its own part of the checkpoint
        sd = hf.state_dict()
        th, tk, cw = (inproc_adapter(i).llm.model for i in range(3))
        assert torch.equal(th.decoder.embed_tokens, sd["thinker.model.embed_tokens.weight"])
        assert torch.equal(th.audio_tower.proj2.weight, sd["thinker.audio_tower.proj2.weight"])
        assert torch.equal(th.visual.merger.fc2.weight, sd["thinker.visual.merger.mlp.2.weight"])
        assert torch.equal(tk.codec_head.weight, sd["talker.codec_head.weight"])
        assert torch.equal(tk.decoder.layers[1].shared_down.weight, sd["talker.model.layers.1.mlp.shared_expert.down_proj.weight"])
        assert torch.equal(tk.code_predictor.lm_heads[2], sd["talker.code_predictor.lm_head.2.weight"])
        assert torch.equal(cw.decoder[1].block[1].conv.weight, sd["code2wav.decoder.1.block.1.conv.weight"])
        assert th.cfg.accept_hidden_layer == 2 and tk.cfg.codec_eos_id == 66
    finally:
        o.close()
    hf.thinker.config.vision_start_token_id = 508          # read by the HF position-id helper, unused for text
    hf.thinker.config.position_id_per_seconds = 25
    for k, v in (("vision_start_token_id", 508), ("audio_start_token_id", 510), ("position_id_per_seconds", 25)):
        if not hasattr(hf.thinker.config, k):              # read by the HF position-id helper, unused for text
            setattr(hf.thinker.config, k, v)
    with torch.no_grad():
        g = hf.thinker.generate(input_ids=torch.tensor([ids]), attention_mask=torch.ones(1, len(ids), dtype=torch.long),
                                max_new_tokens=6, do_sample=False)
    assert mine == g[0, len(ids):].tolist()


def test_mrope_positions_match_hf_rope_index(checkpoint):
    """Text, an image (1x4x6 patches), an audio clip and a video (2x4x4 patches, 2 s per temporal
    grid step) in one prompt: the (t, h, w) position triples equal ``get_rope_index``."""
    from vllm_omni_b200.models.mrope import get_input_positions
    hf, _ = checkpoint
    th = hf.thinker
    th.config.vision_start_token_id, th.config.audio_start_token_id, th.config.position_id_per_seconds = 508, 510, 25
    ids = [506, 10, 508] + [501] * 6 + [509, 11, 510] + [500] * 5 + [511, 12, 508] + [502] * 8 + [509, 13, 14]
    inp = torch.tensor([ids])
    ref, delta = th.get_rope_index(inp, image_grid_thw=torch.tensor([[1, 4, 6]]), video_grid_thw=torch.tensor([[2, 4, 4]]),
                                   attention_mask=torch.ones_like(inp), use_audio_in_video=False,
                                   audio_seqlens=torch.tensor([5]), second_per_grids=torch.tensor([2.0]))
    mine, d = get_input_positions(ids, 501, 502, 500, [(1, 2, 3)], [(2, 2, 2)], seconds_per_grid_t=2.0)
    assert torch.equal(ref[:, 0].long(), mine) and int(delta) == d


# ---------------------------------------------------------------------------- Qwen2.5-Omni
Q25_YAML = YAML.replace("Qwen3OmniMoeForConditionalGeneration", "Qwen2_5OmniForConditionalGeneration") \
    .replace("vllm_omni_b200.models.stage_input_processors.qwen3_omni.thinker2talker",
             "vllm_omni_b200.models.stage_input_processors.qwen2_5_omni.thinker2talker") \
    .replace("vllm_omni_b200.models.stage_input_processors.qwen3_omni.talker2code2wav",
             "vllm_omni_b200.models.stage_input_processors.qwen2_5_omni.talker2code2wav") \
    .replace("stop_token_ids: [66]", "stop_token_ids: [94]")


def test_qwen2_5_omni_hf_checkpoint_through_the_pipeline(tmp_path):
    """``save_pretrained`` of a tiny Qwen2.5-Omni: the three stages load ``thinker.* / talker.* /
    token2wav.*``, the greedy thinker tokens equal transformers', and a waveform comes out."""
    from transformers.models.qwen2_5_omni import modeling_qwen2_5_omni as M
    from transformers.models.qwen2_5_omni.configuration_qwen2_5_omni import Qwen2_5OmniConfig
    from vllm_omni_b200.entrypoints.stage_runtime import inproc_adapter
    torch.manual_seed(0)
    rope = dict(rope_theta=1e6, rope_type="default", mrope_section=[2, 3, 3])
    thinker = dict(
        audio_config=dict(num_mel_bins=16, d_model=32, encoder_layers=1, encoder_attention_heads=2, encoder_ffn_dim=64,
                          output_dim=64, n_window=10, max_source_positions=64),
        vision_config=dict(depth=2, hidden_size=32, intermediate_size=48, num_heads=2, out_hidden_size=64, patch_size=4,
                           window_size=16, fullatt_block_indexes=[1]),
        text_config=dict(vocab_size=512, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, max_position_embeddings=512, rope_parameters=rope),
        audio_token_index=500, image_token_index=501, video_token_index=502)
    talker = dict(vocab_size=96, embedding_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=2,
                  num_attention_heads=2, num_key_value_heads=2, head_dim=16, max_position_embeddings=256, rope_parameters=rope,
                  tts_codec_start_token_id=93, tts_codec_end_token_id=94, tts_codec_pad_token_id=92, tts_codec_mask_token_id=95,
                  tts_text_start_token_id=503, tts_text_end_token_id=504, tts_text_pad_token_id=505)
    t2w = dict(dit_config=dict(hidden_size=32, num_hidden_layers=2, num_attention_heads=2, ff_mult=2, emb_dim=16, head_dim=16,
                               block_size=4, look_ahead_layers=[1], look_backward_layers=[0], repeats=2, num_embeds=97, mel_dim=8,
                               dropout=0.0, enc_emb_dim=8, enc_dim=8, enc_channels=[8, 8, 8, 8, 24],
                               enc_kernel_sizes=[5, 3, 3, 3, 1], enc_dilations=[1, 2, 3, 4, 1], enc_attention_channels=4,
                               enc_res2net_scale=2, enc_se_channels=4, max_position_embeddings=512),
               bigvgan_config=dict(mel_dim=8, upsample_initial_channel=16, resblock_kernel_sizes=[3], resblock_dilation_sizes=[[1, 3, 5]],
                                   upsample_rates=[2, 2], upsample_kernel_sizes=[4, 4]))
    hf = M.Qwen2_5OmniForConditionalGeneration(Qwen2_5OmniConfig(thinker_config=thinker, talker_config=talker,
                                                                 token2wav_config=t2w, enable_audio_output=True))
    for _, p in hf.named_parameters():
        if p.dim() > 1:
            torch.nn.init.normal_(p, 0, 0.05)
    hf = hf.float().eval()
    hf.save_pretrained(str(tmp_path))
    (tmp_path / "stages.yaml").write_text(Q25_YAML)
    ids = [506, 10, 11, 12, 507, 506, 13]
    o = Omni(str(tmp_path), stage_configs_path=str(tmp_path / "stages.yaml"))
    try:
        outs = o.generate([{"prompt_token_ids": ids}])
        mine = list([x for x in outs if x.final_output_type == "text"][0].request_output.outputs[0].token_ids)
        audio = [x for x in outs if x.final_output_type == "audio"][0]
        assert audio.multimodal_output["audio"].dim() == 1
        sd = hf.state_dict()
        th, tk, tw = (inproc_adapter(i).llm.model for i in range(3))
        assert torch.equal(th.audio_tower.proj.weight, sd["thinker.audio_tower.proj.weight"])
        assert torch.equal(th.visual.merge2.weight, sd["thinker.visual.merger.mlp.2.weight"])
        assert torch.equal(tk.codec_embedding, sd["talker.model.embed_tokens.weight"])
        assert torch.equal(tw.dit.proj_out.weight, sd["token2wav.code2wav_dit_model.proj_out.weight"])
        assert torch.equal(tw.vocoder.conv_post.weight, sd["token2wav.code2wav_bigvgan_model.conv_post.weight"])
        assert tk.cfg.codec_eos_id == 94 and tk.cfg.tts_text_bos_id == 503
    finally:
        o.close()
    for k, v in (("vision_start_token_id", 508), ("audio_start_token_id", 510), ("position_id_per_seconds", 25)):
        if not hasattr(hf.thinker.config, k):              # read by the HF position-id helper, unused for text
            setattr(hf.thinker.config, k, v)
    with torch.no_grad():
        g = hf.thinker.generate(input_ids=torch.tensor([ids]), attention_mask=torch.ones(1, len(ids), dtype=torch.long),
                                max_new_tokens=6, do_sample=False)
    assert mine == g[0, len(ids):].tolist()
