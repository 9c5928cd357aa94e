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


# ---------------------------------------------------------------------------- Qwen3-Omni stages
def _init(hf, std=0.05, also=()):
    for n, p in hf.named_parameters():
        if p.dim() > 1 or any(k in n for k in also):
            torch.nn.init.normal_(p, 0, std)
    return hf.float().eval()


def test_qwen3_omni_talker_stage_against_hf():
    """MoE decoder with the shared expert and interleaved MRoPE, resize MLPs, codec head and code
    predictor, all loaded from the ``talker.*`` names of a Hugging Face state dict."""
    M = pytest.importorskip("transformers.models.qwen3_omni_moe.modeling_qwen3_omni_moe")
    from transformers.models.qwen3_omni_moe.configuration_qwen3_omni_moe import Qwen3OmniMoeTalkerConfig
    from vllm_omni_b200.models.qwen3_omni.config import Qwen3OmniConfig
    from vllm_omni_b200.models.qwen3_omni.talker import Qwen3OmniMoeTalker
    torch.manual_seed(0)
    text = dict(vocab_size=96, hidden_size=48, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, head_dim=16, moe_intermediate_size=32, shared_expert_intermediate_size=24,
                num_experts=4, num_experts_per_tok=2, norm_topk_prob=True, max_position_embeddings=512,
                rope_parameters=dict(rope_theta=1e6, rope_type="default", mrope_section=[4, 2, 2], mrope_interleaved=True))
    cp = dict(vocab_size=64, hidden_size=48, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, num_code_groups=4, max_position_embeddings=64)
    hc = Qwen3OmniMoeTalkerConfig(text_config=text, code_predictor_config=cp, thinker_hidden_size=64, num_code_groups=4,
                                  accept_hidden_layer=2, spatial_merge_size=2)
    hf = _init(M.Qwen3OmniMoeTalkerForConditionalGeneration(hc))
    cfg = Qwen3OmniConfig.from_hf({"talker_config": hc.to_dict(), "thinker_config": {}})
    cfg.thinker = Qwen3OmniConfig.tiny().thinker            # width 64 = thinker_hidden_size above
    assert cfg.talker.shared_expert_intermediate_size == 24 and cfg.code_predictor.num_code_groups == 4
    tk = Qwen3OmniMoeTalker(cfg, torch.float32, "cpu")
    sd = {"talker." + k: v for k, v in hf.state_dict().items()}
    assert tk.load_weights(sd.items()) == set(sd)
    T = 11
    x = torch.randn(T, 48)
    pos = torch.stack([torch.arange(T), torch.arange(T) // 2, torch.arange(T) // 3])
    with torch.no_grad():
        ref = hf.model(inputs_embeds=x[None], position_ids=pos[:, None]).last_hidden_state[0]
        b = ModelBatch(torch.zeros(T, dtype=torch.long), pos, torch.full((T,), -1, dtype=torch.int32),
                       [PrefillSeg(0, T, 0, None)], input_embeds=x)
        h, _ = tk.decoder(b, None)
        assert (h - ref).abs().max().item() < 1e-4
        assert (tk.compute_logits(h) - hf.codec_head(ref)).abs().max().item() < 1e-4
        y = torch.randn(5, 64)
        assert (tk.text_projection(y) - hf.text_projection(y)).abs().max().item() < 1e-5
        assert (tk.hidden_projection(y) - hf.hidden_projection(y)).abs().max().item() < 1e-5
        s = torch.randn(2, 3, 48)                       # talker hidden, code 0, code 1 -> logits of code 2
        r = hf.code_predictor(inputs_embeds=s)
        mine = torch.nn.functional.linear(tk.code_predictor._forward_seq(s), tk.code_predictor.lm_heads[1])
        assert (mine - r.logits).abs().max().item() < 1e-4


def test_qwen3_omni_code2wav_against_hf():
    M = pytest.importorskip("transformers.models.qwen3_omni_moe.modeling_qwen3_omni_moe")
    from transformers.models.qwen3_omni_moe.configuration_qwen3_omni_moe import Qwen3OmniMoeCode2WavConfig
    from vllm_omni_b200.models.qwen3_omni.code2wav import Qwen3OmniCode2Wav
    from vllm_omni_b200.models.qwen3_omni.config import Qwen3OmniConfig
    torch.manual_seed(0)
    hc = Qwen3OmniMoeCode2WavConfig(codebook_size=64, hidden_size=32, num_attention_heads=2, num_key_value_heads=2,
                                    sliding_window=5, intermediate_size=64, num_hidden_layers=2, num_quantizers=4,
                                    upsample_rates=[4, 2], upsampling_ratios=[2], decoder_dim=32, max_position_embeddings=512)
    hf = _init(M.Qwen3OmniMoeCode2Wav(hc), 0.08, also=("alpha", "beta", "gamma", "scale", "bias"))
    cfg = Qwen3OmniConfig.from_hf({"code2wav_config": hc.to_dict()})
    m = Qwen3OmniCode2Wav(cfg, torch.float32, "cpu")
    sd = {"code2wav." + k: v for k, v in hf.state_dict().items()}
    assert m.load_weights(sd.items()) == set(sd)
    codes = torch.randint(0, 64, (2, 4, 13))
    with torch.no_grad():
        ref, out = hf(codes)[:, 0], m.decode(codes)
        assert ref.shape == out.shape and 0.05 < ref.abs().max().item() < 0.99        # not saturated by the clamp
        assert (ref - out).abs().max().item() < 1e-5
        r2 = hf.chunked_decode(codes, chunk_size=5, left_context_size=2)[:, 0]
        o2 = m.chunked_decode(codes, 5, 2)
        assert r2.shape == o2.shape and (r2 - o2).abs().max().item() < 1e-5


def _init_all(hf):
    for n, p in hf.named_parameters():
        if p.dim() > 1:
            torch.nn.init.normal_(p, 0, 0.05)
        else:
            torch.nn.init.normal_(p, 0.5 if ("norm" in n or "ln" in n) else 0.0, 0.1)
    return hf.float().eval()


def test_qwen3_omni_audio_tower_against_hf():
    """Chunked conv stem, per-chunk positions and block-diagonal windows.  The eager attention path
    of the HF module drops ``cu_seqlens``; its own block-diagonal mask is handed to the layers so
    that the oracle has the windowed semantics of its variable-length attention path."""
    M = pytest.importorskip("transformers.models.qwen3_omni_moe.modeling_qwen3_omni_moe")
    from transformers.models.qwen3_omni_moe.configuration_qwen3_omni_moe import Qwen3OmniMoeAudioEncoderConfig
    from vllm_omni_b200.models.qwen3_omni.config import Qwen3OmniConfig
    from vllm_omni_b200.models.qwen3_omni.encoders import AudioEncoder
    torch.manual_seed(0)
    ac = Qwen3OmniMoeAudioEncoderConfig(num_mel_bins=16, d_model=32, encoder_layers=2, encoder_attention_heads=2,
                                        encoder_ffn_dim=64, downsample_hidden_size=8, output_dim=24, n_window=50,
                                        n_window_infer=200, max_source_positions=64, conv_chunksize=500)
    hf = _init_all(M.Qwen3OmniMoeAudioEncoder(ac))
    cfg = Qwen3OmniConfig.from_hf({"thinker_config": {"audio_config": ac.to_dict()}})
    enc = AudioEncoder(cfg.audio, torch.float32, "cpu")
    sd = hf.state_dict()
    assert enc.load_weights(sd.items()) == set(sd)

    def windowed(mel, T):
        origs = [layer.forward for layer in hf.layers]
        for layer, orig in zip(hf.layers, origs):
            layer.forward = lambda hs, cu, attention_mask=None, _o=orig, **kw: _o(
                hs, cu, attention_mask=hf._prepare_attention_mask(hs, cu), **kw)
        try:
            return hf(mel, feature_lens=torch.tensor([T])).last_hidden_state
        finally:
            for layer, orig in zip(hf.layers, origs):
                layer.forward = orig

    for T in (530, 100, 37, 300):          # several chunks + short tail, one full chunk, one short chunk, exact chunks
        mel = torch.randn(16, T)
        with torch.no_grad():
            ref, out = windowed(mel, T), enc(mel)
        assert out.shape == ref.shape and out.shape[0] == enc.output_length(T)
        assert (ref - out).abs().max().item() < 1e-5, T


def test_qwen3_omni_vision_tower_against_hf():
    M = pytest.importorskip("transformers.models.qwen3_omni_moe.modeling_qwen3_omni_moe")
    from transformers.models.qwen3_omni_moe.configuration_qwen3_omni_moe import Qwen3OmniMoeVisionEncoderConfig
    from vllm_omni_b200.models.qwen3_omni.config import Qwen3OmniConfig
    from vllm_omni_b200.models.qwen3_omni.encoders import VisionEncoder
    torch.manual_seed(0)
    vc = Qwen3OmniMoeVisionEncoderConfig(depth=3, hidden_size=32, num_heads=2, intermediate_size=64, patch_size=4,
                                         temporal_patch_size=2, spatial_merge_size=2, in_channels=3, out_hidden_size=24,
                                         num_position_embeddings=16, deepstack_visual_indexes=[0, 2])
    hf = _init_all(M.Qwen3OmniMoeVisionEncoder(vc))
    cfg = Qwen3OmniConfig.from_hf({"thinker_config": {"vision_config": vc.to_dict()}})
    enc = VisionEncoder(cfg.vision, torch.float32, "cpu")
    sd = hf.state_dict()
    assert enc.load_weights(sd.items()) == set(sd)
    gt, gh, gw = 2, 6, 4
    patches = torch.randn(gt * gh * gw, 3 * 2 * 4 * 4)
    with torch.no_grad():
        r = hf(patches, grid_thw=torch.tensor([[gt, gh, gw]]))
        out, grid, deep = enc.forward_patches(patches, (gt, gh, gw))
    assert grid == (2, 3, 2) and (r.pooler_output - out).abs().max().item() < 1e-5
    assert len(deep) == 2
    for a, b in zip(r.deepstack_features, deep):
        assert (a - b).abs().max().item() < 1e-5
    # pixel entry point: frames [T, C, H, W] are cut into the same patch order
    px = torch.randn(4, 3, 24, 16)
    tp, p, m = 2, 4, 2
    x = px.reshape(2, tp, 3, 3, m, p, 2, m, p).permute(0, 3, 6, 4, 7, 2, 1, 5, 8).reshape(2 * 6 * 4, -1)
    with torch.no_grad():
        o1, g1, _ = enc(px)
        o2 = hf(x, grid_thw=torch.tensor([[2, 6, 4]])).pooler_output
    assert g1 == (2, 3, 2) and (o1 - o2).abs().max().item() < 1e-5


def test_qwen3_omni_thinker_text_with_deepstack_against_hf():
    M = pytest.importorskip("transformers.models.qwen3_omni_moe.modeling_qwen3_omni_moe")
    from transformers.models.qwen3_omni_moe.configuration_qwen3_omni_moe import Qwen3OmniMoeTextConfig
    torch.manual_seed(0)
    tc = Qwen3OmniMoeTextConfig(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=3,
                                num_attention_heads=4, num_key_value_heads=2, head_dim=16, moe_intermediate_size=32,
                                num_experts=4, num_experts_per_tok=2, norm_topk_prob=True, max_position_embeddings=512,
                                decoder_sparse_step=1, mlp_only_layers=[],
                                rope_parameters=dict(rope_theta=1e6, rope_type="default", mrope_section=[4, 2, 2],
                                                     mrope_interleaved=True))
    hf = _init(M.Qwen3OmniMoeThinkerTextModel(tc))
    cfg = DecoderConfig.from_dict(tc.to_dict())
    assert cfg.mrope_section == (4, 2, 2) and cfg.mrope_interleaved and cfg.num_experts == 4
    m = QwenDecoderModel(cfg, torch.float32, "cpu", with_lm_head=False)
    sd = {"model." + k: v for k, v in hf.state_dict().items()}
    assert m.load_weights(sd.items()) == set(sd)
    T = 14
    ids = torch.randint(0, 128, (T,))
    pos = torch.stack([torch.arange(T), torch.arange(T) // 2, (torch.arange(T) * 2) % 5])
    vis = torch.zeros(T, dtype=torch.bool)
    vis[3:9] = True
    feats = [torch.randn(6, 64) for _ in range(2)]
    with torch.no_grad():
        ref = hf(input_ids=ids[None], position_ids=pos[:, None], visual_pos_masks=vis[None],
                 deepstack_visual_embeds=feats).last_hidden_state[0]
        dense = []
        for f in feats:
            d = torch.zeros(T, 64)
            d[vis] = f
            dense.append(d)
        b = ModelBatch(ids, pos, torch.full((T,), -1, dtype=torch.int32), [PrefillSeg(0, T, 0, None)])
        out, _ = m(b, None, deepstack=dense)
    assert (out - ref).abs().max().item() < 1e-4 * max(1.0, ref.abs().max().item())


def test_qwen_image_prompt_encoder_against_hf_qwen2_5_vl():
    """Packed (padding-free) prompt encoding equals the HF model's last hidden states behind the
    34-token template head, for prompts of different lengths."""
    from vllm_omni_b200.diffusion.models.qwen_image.text_encoder import QwenVLTextEncoder, text_config_from_hf
    from vllm_omni_b200.engine.tokenizer import ByteTokenizer
    torch.manual_seed(0)
    hc = transformers.Qwen2_5_VLConfig(
        text_config=dict(vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, max_position_embeddings=2048,
                         rope_parameters=dict(rope_theta=1e6, rope_type="default", mrope_section=[2, 3, 3])),
        vision_config=dict(depth=1, hidden_size=32, intermediate_size=64, num_heads=2, out_hidden_size=64, patch_size=4,
                           fullatt_block_indexes=[0]))
    hf = transformers.Qwen2_5_VLForConditionalGeneration(hc).float().eval()
    enc = QwenVLTextEncoder(text_config_from_hf(hc.to_dict()), ByteTokenizer(), torch.float32, "cpu")
    sd = hf.state_dict()
    want = {k for k in sd if "visual" not in k and not k.startswith("lm_head")}
    assert enc.load_weights(sd.items()) == want
    prompts = ["a cat on a mat", "a much longer prompt about a dog that sits under the old tree"]
    states, mask = enc(prompts)
    tok = ByteTokenizer()
    seqs = [tok.encode(enc.template.format(p)) for p in prompts]
    L = max(len(s) for s in seqs)
    ids, am = torch.zeros(2, L, dtype=torch.long), torch.zeros(2, L, dtype=torch.long)
    for i, s in enumerate(seqs):
        ids[i, :len(s)], am[i, :len(s)] = torch.tensor(s), 1
    with torch.no_grad():
        ref = hf(input_ids=ids, attention_mask=am, output_hidden_states=True).hidden_states[-1]
    assert states.shape == (2, L - 34, 64)
    for i, s in enumerate(seqs):
        n = len(s) - 34
        assert int(mask[i].sum()) == n and states[i, n:].abs().sum() == 0
        assert (states[i, :n] - ref[i, 34:len(s)]).abs().max().item() < 1e-4
    short, _ = enc(prompts, max_sequence_length=50)
    assert short.shape[1] == 50 and torch.equal(short, states[:, :50])


def test_z_image_caption_encoder_takes_second_to_last_layer():
    from vllm_omni_b200.diffusion.models.z_image.text_encoder import QwenCaptionEncoder
    from vllm_omni_b200.engine.tokenizer import ByteTokenizer
    torch.manual_seed(0)
    hf = transformers.Qwen3ForCausalLM(transformers.Qwen3Config(**{**BASE, "vocab_size": 300, "num_hidden_layers": 3}, head_dim=32)).float().eval()
    enc = QwenCaptionEncoder(DecoderConfig.from_dict(hf.config.to_dict()), ByteTokenizer(), torch.float32, "cpu")
    sd = hf.state_dict()
    assert enc.load_weights(sd.items()) == {k for k in sd if not k.startswith("lm_head")}
    prompts = ["a lighthouse at dusk", "fog"]
    states, mask = enc(prompts)
    for i, p in enumerate(prompts):
        ids = torch.tensor([enc._ids(p)])
        with torch.no_grad():
            ref = hf(input_ids=ids, output_hidden_states=True).hidden_states[-2][0]
        n = ids.shape[1]
        assert int(mask[i].sum()) == n and (states[i, :n] - ref).abs().max().item() < 1e-4


@pytest.mark.parametrize("grid", [(1, 8, 12), (2, 6, 10), (1, 4, 4)])
def test_qwen2_5_vl_vision_tower_against_hf(grid):
    """Window attention (ragged windows at the right / bottom edge), full-attention blocks, 2-D rotary
    embedding, window re-ordering and its inverse, SwiGLU blocks, patch merger."""
    from vllm_omni_b200.models.qwen2_5_vl_vision import Qwen25VisionConfig, Qwen25VisionTower
    torch.manual_seed(0)
    hc = transformers.Qwen2_5_VLConfig(
        text_config=dict(vocab_size=64, hidden_size=64, intermediate_size=96, num_hidden_layers=1, num_attention_heads=4,
                         num_key_value_heads=2),
        vision_config=dict(depth=3, hidden_size=32, intermediate_size=48, num_heads=2, out_hidden_size=64, patch_size=4,
                           window_size=24, fullatt_block_indexes=[1]))
    hf = _init_all(transformers.Qwen2_5_VLForConditionalGeneration(hc)).model.visual
    tower = Qwen25VisionTower(Qwen25VisionConfig.from_dict(hc.vision_config.to_dict()), torch.float32, "cpu")
    sd = hf.state_dict()
    assert tower.load_weights(sd.items()) == set(sd)
    gt, gh, gw = grid
    patches = torch.randn(gt * gh * gw, 3 * 2 * 4 * 4)
    with torch.no_grad():
        ref = hf(patches, grid_thw=torch.tensor([[gt, gh, gw]])).pooler_output
        out, g = tower.forward_patches(patches, grid)
    assert g == (gt, gh // 2, gw // 2) and out.shape == ref.shape
    assert (out - ref).abs().max().item() < 1e-4 * max(1.0, ref.abs().max().item())


class _SlotTokenizer:
    """Bytes as ids, plus single ids for the three vision markers."""
    MARK = {"<|vision_start|>": 290, "<|image_pad|>": 291, "<|vision_end|>": 292}

    def encode(self, text, add_special_tokens=False):
        import re
        out = []
        for part in re.split("(" + "|".join(re.escape(k) for k in self.MARK) + ")", text):
            out.extend([self.MARK[part]] if part in self.MARK else list(part.encode()))
        return out


def test_qwen_image_edit_prompt_encoder_with_an_image_against_hf():
    """Instruction + condition image through the vision tower and the language model with (t, h, w)
    rotary positions: the states behind the template head equal the HF model's."""
    from vllm_omni_b200.diffusion.models.qwen_image.text_encoder import QwenVLTextEncoder, text_config_from_hf
    from vllm_omni_b200.models.qwen2_5_vl_vision import Qwen25VisionConfig
    torch.manual_seed(0)
    hc = transformers.Qwen2_5_VLConfig(
        text_config=dict(vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, max_position_embeddings=2048,
                         rope_parameters=dict(rope_theta=1e6, rope_type="default", mrope_section=[2, 3, 3])),
        vision_config=dict(depth=2, hidden_size=32, intermediate_size=48, num_heads=2, out_hidden_size=64, patch_size=4,
                           window_size=16, fullatt_block_indexes=[1]),
        image_token_id=291, vision_start_token_id=290, vision_end_token_id=292, video_token_id=293)
    hf = _init_all(transformers.Qwen2_5_VLForConditionalGeneration(hc))
    enc = QwenVLTextEncoder(text_config_from_hf(hc.to_dict()), _SlotTokenizer(), torch.float32, "cpu",
                            vision_config=Qwen25VisionConfig.from_dict(hc.vision_config.to_dict()), image_token_id=291)
    assert enc.cfg.mrope_section == (2, 3, 3)
    sd = hf.state_dict()
    assert enc.load_weights(sd.items()) == {k for k in sd if not k.startswith("lm_head")}
    grid = (1, 6, 4)                                            # 24 patches -> 6 merged tokens
    patches = torch.randn(24, 3 * 2 * 4 * 4)
    template, drop = "<|im_start|>user\n{}<|im_end|>\n<|im_start|>assistant\n", 5
    states, mask = enc.encode_with_images(["make it blue"], [[]], template=template, drop_tokens=drop,
                                          patches=[[(patches, grid)]])
    tok = _SlotTokenizer()
    ids = tok.encode(template.format("<|vision_start|><|image_pad|><|vision_end|>make it blue"))
    i = ids.index(291)
    ids = ids[:i] + [291] * 6 + ids[i + 1:]
    inp = torch.tensor([ids])
    with torch.no_grad():
        # positions: (t, h, w) of the original Qwen2.5-VL rule (an image keeps t = its start index), the one
        # the Qwen3-Omni test checks against ``get_rope_index``; this release's Qwen2.5-VL helper scales t
        from vllm_omni_b200.models.mrope import get_input_positions
        pos, _ = get_input_positions(ids, 291, -1, -2, [(1, 3, 2)], [])
        ref = hf(input_ids=inp, attention_mask=torch.ones_like(inp), pixel_values=patches,
                 image_grid_thw=torch.tensor([list(grid)]), position_ids=pos[:, None],
                 output_hidden_states=True).hidden_states[-1][0]
    n = len(ids) - drop
    assert states.shape == (1, n, 64) and int(mask.sum()) == n
    assert (states[0] - ref[drop:]).abs().max().item() < 1e-4 * max(1.0, ref.abs().max().item())


def test_qwen2_5_omni_audio_tower_against_hf():
    M = pytest.importorskip("transformers.models.qwen2_5_omni.modeling_qwen2_5_omni")
    from transformers.models.qwen2_5_omni.configuration_qwen2_5_omni import Qwen2_5OmniAudioEncoderConfig
    from vllm_omni_b200.models.qwen2_5_omni.audio import Qwen25AudioConfig, Qwen25AudioEncoder
    torch.manual_seed(0)
    ac = Qwen2_5OmniAudioEncoderConfig(num_mel_bins=16, d_model=32, encoder_layers=2, encoder_attention_heads=2,
                                       encoder_ffn_dim=64, output_dim=24, n_window=10, max_source_positions=64)
    hf = _init_all(M.Qwen2_5OmniAudioEncoder(ac))
    enc = Qwen25AudioEncoder(Qwen25AudioConfig.from_dict(ac.to_dict()), torch.float32, "cpu")
    sd = hf.state_dict()
    assert enc.load_weights(sd.items()) == set(sd)
    for T in (53, 20, 7, 40):              # chunks of 20 frames: ragged tail, one chunk, short chunk, exact
        mel = torch.randn(16, T)
        full, tail = divmod(T, 20)
        after = full * 10 + ((tail - 1) // 2 + 1 if tail else 0)
        with torch.no_grad():
            ref = hf(mel, feature_lens=torch.tensor([T]), aftercnn_lens=torch.tensor([after])).last_hidden_state
            out = enc(mel)
        assert out.shape == ref.shape and out.shape[0] == enc.output_length(T), T
        assert (ref - out).abs().max().item() < 1e-5, T


def test_qwen2_5_omni_talker_against_hf():
    """Codec embedding table in the thinker width, ``thinker_to_talker_proj``, dense Qwen2 decoder with
    MRoPE, codec head — loaded from the ``talker.*`` names."""
    M = pytest.importorskip("transformers.models.qwen2_5_omni.modeling_qwen2_5_omni")
    from transformers.models.qwen2_5_omni.configuration_qwen2_5_omni import Qwen2_5OmniTalkerConfig
    from vllm_omni_b200.models.qwen2_5_omni.config import Qwen25OmniConfig
    from vllm_omni_b200.models.qwen2_5_omni.talker import Qwen25OmniTalker
    torch.manual_seed(0)
    tc = Qwen2_5OmniTalkerConfig(vocab_size=96, embedding_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=2,
                                 num_attention_heads=2, num_key_value_heads=2, head_dim=16, max_position_embeddings=256,
                                 rope_parameters=dict(rope_theta=1e6, rope_type="default", mrope_section=[2, 3, 3]),
                                 tts_codec_start_token_id=93, tts_codec_end_token_id=94, tts_codec_pad_token_id=92)
    hf = _init_all(M.Qwen2_5OmniTalkerForConditionalGeneration(tc))
    cfg = Qwen25OmniConfig.from_hf({"talker_config": tc.to_dict(), "thinker_config": {}})
    assert cfg.talker_embedding_size == 64 and cfg.talker.mrope_section == (2, 3, 3) and cfg.codec_bos_id == 93
    tk = Qwen25OmniTalker(cfg, torch.float32, "cpu")
    sd = {"talker." + k: v for k, v in hf.state_dict().items()}
    assert tk.load_weights(sd.items()) == set(sd)
    T = 9
    x = torch.randn(T, 64)
    pos = torch.stack([torch.arange(T), torch.arange(T) // 2, torch.arange(T) // 3])
    with torch.no_grad():
        ref = hf(inputs_embeds=x[None].clone(), position_ids=pos[:, None]).logits[0]
        b = ModelBatch(torch.zeros(T, dtype=torch.long), pos, torch.full((T,), -1, dtype=torch.int32),
                       [PrefillSeg(0, T, 0, None)], input_embeds=tk.thinker_to_talker_proj(x))
        h, _ = tk.decoder(b, None)
        out = tk.codec_head(h)
    assert (out - ref).abs().max().item() < 1e-4 * max(1.0, ref.abs().max().item())
    assert torch.isinf(tk.compute_logits(h)[:, 93]).all()            # the start marker cannot be sampled


def test_qwen2_5_omni_token2wav_against_hf():
    """DiT (ECAPA speaker encoder, first-head rotary, block-local attention, guided velocity), the
    sampled mel spectrogram and the BigVGAN waveform, from the ``token2wav.*`` names."""
    M = pytest.importorskip("transformers.models.qwen2_5_omni.modeling_qwen2_5_omni")
    from transformers.models.qwen2_5_omni.configuration_qwen2_5_omni import (Qwen2_5OmniBigVGANConfig, Qwen2_5OmniDiTConfig,
                                                                            Qwen2_5OmniToken2WavConfig)
    from vllm_omni_b200.models.qwen2_5_omni.config import Qwen25OmniConfig
    from vllm_omni_b200.models.qwen2_5_omni.token2wav import Qwen25OmniToken2Wav
    torch.manual_seed(0)
    dc = dict(hidden_size=32, num_hidden_layers=3, num_attention_heads=2, ff_mult=2, emb_dim=16, head_dim=16, block_size=4,
              look_ahead_layers=[1], look_backward_layers=[0, 2], repeats=2, num_embeds=97, mel_dim=8, dropout=0.0,
              enc_emb_dim=8, enc_dim=8, enc_channels=[8, 8, 8, 8, 24], enc_kernel_sizes=[5, 3, 3, 3, 1], enc_dilations=[1, 2, 3, 4, 1],
              enc_attention_channels=4, enc_res2net_scale=2, enc_se_channels=4, max_position_embeddings=512)
    bc = dict(mel_dim=8, upsample_initial_channel=16, resblock_kernel_sizes=[3, 5], resblock_dilation_sizes=[[1, 3, 5], [1, 3, 5]],
              upsample_rates=[2, 2], upsample_kernel_sizes=[4, 4])
    hc = Qwen2_5OmniToken2WavConfig(dit_config=dc, bigvgan_config=bc)
    hf = M.Qwen2_5OmniToken2WavModel(hc)
    for n, p in hf.named_parameters():
        torch.nn.init.normal_(p, 0, 0.15 if p.dim() > 1 else 0.05)
    hf = hf.float().eval()
    cfg = Qwen25OmniConfig.from_hf({"token2wav_config": hc.to_dict(), "thinker_config": {}})
    assert cfg.dit.look_backward_layers == (0, 2) and cfg.bigvgan.resblock_dilation_sizes == ((1, 3, 5), (1, 3, 5))
    m = Qwen25OmniToken2Wav(cfg, torch.float32, "cpu")
    sd = {"token2wav." + k: v for k, v in hf.state_dict().items()}
    assert m.load_weights(sd.items()) == set(sd)
    B, Tc = 1, 10
    codes = torch.randint(1, 90, (B, Tc))
    xvec, ref = torch.randn(B, 8), torch.randn(B, 11, 8)
    x = torch.randn(B, 2 * Tc, 8)
    xv = xvec.unsqueeze(1).repeat(1, 2 * Tc, 1)
    with torch.no_grad():
        a = hf.code2wav_dit_model(hidden_states=x, condition_vector=ref, speaker_embedding=xv, quantized_code=codes,
                                  time_step=torch.tensor(0.37), apply_cfg=True)
        b = m.dit(x, ref, xv, codes, torch.tensor(0.37), apply_cfg=True)
        assert a.shape == b.shape == (2, 2 * Tc, 8) and (a - b).abs().max().item() < 1e-4 * max(1.0, a.abs().max().item())
        # the whole sampler from the same noise
        torch.manual_seed(5)
        mel_ref = hf.code2wav_dit_model.sample(xvec, ref, codes, num_steps=4, guidance_scale=0.5, sway_coefficient=-1.0)
        torch.manual_seed(5)
        noise = torch.randn(B, 2 * Tc, 8)
        mel = m.dit.sample(codes, xvec, ref, num_steps=4, guidance_scale=0.5, sway=-1.0, noise=noise)
        assert mel.shape == mel_ref.shape == (B, 8, 2 * Tc)
        assert (mel - mel_ref).abs().max().item() < 1e-3 * max(1.0, mel_ref.abs().max().item())
        wav_ref = hf.code2wav_bigvgan_model(mel_ref)
        wav = m.vocoder(mel_ref)[0]
        assert wav.shape == wav_ref.shape == (2 * Tc * 4,) and (wav - wav_ref).abs().max().item() < 1e-4
        assert 0.01 < wav_ref.abs().max().item()
