"""T5 and CLIP prompt encoders against transformers (random weights, fp32, CPU): state dicts load by
Hugging Face names and the outputs agree."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from vllm_omni_b200.diffusion.models.text_encoders.clip import CLIPTextConfig, CLIPTextEncoder
from vllm_omni_b200.diffusion.models.text_encoders.t5 import T5Config, T5Encoder, relative_position_bucket


def _init(m, std=0.08):
    for n, p in m.named_parameters():
        if p.dim() > 1:
            torch.nn.init.normal_(p, 0, std)
        else:
            torch.nn.init.normal_(p, 0.7 if "norm" in n else 0.0, 0.1)
    return m.float().eval()


@pytest.mark.parametrize("ff", ["relu", "gated-gelu"])
def test_t5_encoder_against_hf(ff):
    torch.manual_seed(0)
    hc = transformers.T5Config(vocab_size=200, d_model=48, d_kv=8, d_ff=96, num_layers=3, num_heads=4,
                               relative_attention_num_buckets=8, relative_attention_max_distance=20, feed_forward_proj=ff)
    hf = _init(transformers.T5EncoderModel(hc))
    cfg = T5Config.from_dict(hc.to_dict())
    assert cfg.gated == (ff != "relu")
    m = T5Encoder(cfg, torch.float32, "cpu")
    sd = hf.state_dict()
    loaded = m.load_weights(sd.items())
    assert loaded == set(sd), set(sd) - loaded
    ids = torch.randint(0, 200, (2, 37))
    mask = torch.ones(2, 37, dtype=torch.long)
    mask[1, 25:] = 0
    with torch.no_grad():
        ref = hf(ids).last_hidden_state
        out = m(ids)
        assert (ref - out).abs().max().item() < 2e-5 * max(1.0, ref.abs().max().item())
        ref = hf(ids, attention_mask=mask).last_hidden_state
        out = m(ids, mask)
        assert (ref - out)[mask.bool()].abs().max().item() < 2e-5 * max(1.0, ref.abs().max().item())


def test_umt5_encoder_against_hf():
    """Wan's text encoder: T5 with one relative-position table per block."""
    torch.manual_seed(0)
    hc = transformers.UMT5Config(vocab_size=200, d_model=48, d_kv=8, d_ff=96, num_layers=3, num_heads=4,
                                 relative_attention_num_buckets=8, relative_attention_max_distance=20, feed_forward_proj="gated-gelu")
    hf = _init(transformers.UMT5EncoderModel(hc))
    cfg = T5Config.from_dict(hc.to_dict())
    assert cfg.per_layer_bias and cfg.gated
    m = T5Encoder(cfg, torch.float32, "cpu")
    sd = hf.state_dict()
    assert m.load_weights(sd.items()) == set(sd)
    assert not torch.equal(m.rel_bias[0], m.rel_bias[2])
    ids = torch.randint(0, 200, (2, 21))
    mask = torch.ones(2, 21, dtype=torch.long)
    mask[0, 13:] = 0
    with torch.no_grad():
        ref = hf(ids, attention_mask=mask).last_hidden_state
        out = m(ids, mask)
    assert (ref - out)[mask.bool()].abs().max().item() < 2e-5 * max(1.0, ref.abs().max().item())


def test_relative_position_buckets_cover_both_signs():
    rel = torch.arange(-40, 41)
    b = relative_position_bucket(rel, 8, 20)
    assert b.min().item() == 0 and b.max().item() == 7
    assert (b[rel <= 0] < 4).all() and (b[rel > 0] >= 4).all()
    assert b[rel == -1].item() == 1 and b[rel == 1].item() == 5          # small distances are exact


@pytest.mark.parametrize("proj,act,eos", [(False, "quick_gelu", 2), (True, "gelu", 150)])
def test_clip_text_encoder_against_hf(proj, act, eos):
    torch.manual_seed(1)
    hc = transformers.CLIPTextConfig(vocab_size=160, hidden_size=32, intermediate_size=64, num_hidden_layers=3,
                                     num_attention_heads=4, max_position_embeddings=20, hidden_act=act, projection_dim=24,
                                     eos_token_id=eos, bos_token_id=0, pad_token_id=1)
    cls = transformers.CLIPTextModelWithProjection if proj else transformers.CLIPTextModel
    hf = _init(cls(hc))
    d = hc.to_dict()
    d["architectures"] = [cls.__name__]
    cfg = CLIPTextConfig.from_dict(d)
    assert (cfg.projection_dim is not None) == proj
    m = CLIPTextEncoder(cfg, torch.float32, "cpu")
    sd = hf.state_dict()
    loaded = m.load_weights(sd.items())
    assert loaded == set(sd), set(sd) - loaded
    ids = torch.randint(3, 140, (2, 20))
    ids[0, 11], ids[1, 19] = (159, 159) if eos == 2 else (eos, eos)      # end-of-text: largest id / the configured id
    with torch.no_grad():
        r = hf(ids, output_hidden_states=True)
        last, pooled, pen = m(ids)
    assert (r.last_hidden_state - last).abs().max().item() < 2e-5
    assert (r.hidden_states[-2] - pen).abs().max().item() < 2e-5
    ref_pooled = r.text_embeds if proj else r.pooler_output
    assert (ref_pooled - pooled).abs().max().item() < 2e-5


# ----------------------------------------------------------------------------- diffusers folders with encoders
def _tokenizer_dir(path, max_len, eos="</s>", pad="<pad>"):
    from tokenizers import Tokenizer, models, pre_tokenizers, processors
    words = [pad, eos, "<unk>"] + [chr(c) for c in range(97, 123)] + ["a red cube", "on", "table", "blurry", "the"]
    tok = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    tok.post_processor = processors.TemplateProcessing(single=f"$A {eos}", special_tokens=[(eos, 1)])
    fast = transformers.PreTrainedTokenizerFast(tokenizer_object=tok, pad_token=pad, eos_token=eos, unk_token="<unk>",
                                                model_max_length=max_len)
    fast.save_pretrained(str(path))


def _save_clip(path, hidden, proj, with_projection):
    hc = transformers.CLIPTextConfig(vocab_size=40, hidden_size=hidden, intermediate_size=2 * hidden, num_hidden_layers=2,
                                     num_attention_heads=2, max_position_embeddings=77, projection_dim=proj, eos_token_id=1,
                                     bos_token_id=0, pad_token_id=0)
    cls = transformers.CLIPTextModelWithProjection if with_projection else transformers.CLIPTextModel
    hf = _init(cls(hc))
    hf.save_pretrained(str(path))
    return hf


def _save_t5(path, d_model):
    hc = transformers.T5Config(vocab_size=40, d_model=d_model, d_kv=8, d_ff=2 * d_model, num_layers=2, num_heads=2,
                               relative_attention_num_buckets=8, relative_attention_max_distance=16, feed_forward_proj="gated-gelu")
    hf = _init(transformers.T5EncoderModel(hc))
    hf.save_pretrained(str(path))
    return hf


SMALL_KL = dict(block_out_channels=(8, 16, 16, 16), layers_per_block=1, norm_num_groups=4)


def _load(d, **kw):
    from vllm_omni_b200.diffusion.loader import DiffusersPipelineLoader
    from vllm_omni_b200.entrypoints.omni_diffusion import build_diffusion_config
    cfg = build_diffusion_config(str(d), dtype="float32", vae_config=SMALL_KL, output_type="latent", **kw)
    return DiffusersPipelineLoader(cfg).load_model("cpu")


def test_flux_folder_attaches_clip_and_t5(tmp_path):
    import json
    pytest.importorskip("tokenizers")
    torch.manual_seed(0)
    d = tmp_path
    (d / "model_index.json").write_text(json.dumps({"_class_name": "FluxPipeline"}))
    (d / "transformer").mkdir()
    (d / "transformer" / "config.json").write_text(json.dumps(dict(
        _class_name="FluxTransformer2DModel", num_layers=1, num_single_layers=1, attention_head_dim=32, num_attention_heads=2,
        joint_attention_dim=48, pooled_projection_dim=24, axes_dims_rope=[8, 12, 12], in_channels=64, out_channels=16)))
    clip = _save_clip(d / "text_encoder", 24, 24, False)
    t5 = _save_t5(d / "text_encoder_2", 48)
    _tokenizer_dir(d / "tokenizer", 77)
    _tokenizer_dir(d / "tokenizer_2", 512)
    pipe = _load(d)
    from vllm_omni_b200.diffusion.models.text_encoders.clip import CLIPPromptEncoder
    from vllm_omni_b200.diffusion.models.text_encoders.t5 import T5PromptEncoder
    assert isinstance(pipe.text_encoder, T5PromptEncoder) and isinstance(pipe.pooled_encoder, CLIPPromptEncoder)
    texts = ["a red cube on the table", "blurry"]
    tok2 = transformers.AutoTokenizer.from_pretrained(str(d / "tokenizer_2"))
    tok1 = transformers.AutoTokenizer.from_pretrained(str(d / "tokenizer"))
    with torch.no_grad():
        ids = tok2(texts, padding="max_length", max_length=32, truncation=True, return_tensors="pt").input_ids
        ref = t5(ids).last_hidden_state
        pe, mask = pipe.text_encoder(texts, "cpu", torch.float32, 32)
        assert pe.shape == (2, 32, 48) and mask.all() and (pe - ref).abs().max().item() < 2e-5 * max(1.0, ref.abs().max().item())
        ids = tok1(texts, padding="max_length", max_length=77, truncation=True, return_tensors="pt").input_ids
        ref = clip(ids).pooler_output
        pooled = pipe.pooled_encoder(texts, "cpu", torch.float32)[0][:, 0]
        assert (pooled - ref).abs().max().item() < 2e-5
    # and the pipeline runs with them
    from vllm_omni_b200.diffusion.request import OmniDiffusionRequest
    from vllm_omni_b200.inputs import OmniDiffusionSamplingParams
    sp = OmniDiffusionSamplingParams(height=32, width=32, num_inference_steps=2, seed=1, output_type="latent", max_sequence_length=32)
    out = pipe(OmniDiffusionRequest(prompts=[texts[0]], sampling_params=sp, request_ids=["r"]))
    assert torch.isfinite(out.output).all()


def test_sd3_folder_builds_the_joint_conditioning(tmp_path):
    import json
    pytest.importorskip("tokenizers")
    torch.manual_seed(0)
    d = tmp_path
    (d / "model_index.json").write_text(json.dumps({"_class_name": "StableDiffusion3Pipeline"}))
    (d / "transformer").mkdir()
    (d / "transformer" / "config.json").write_text(json.dumps(dict(
        _class_name="SD3Transformer2DModel", num_layers=2, attention_head_dim=16, num_attention_heads=2, joint_attention_dim=64,
        caption_projection_dim=32, pooled_projection_dim=28, in_channels=16, patch_size=2, out_channels=16, sample_size=16,
        pos_embed_max_size=16)))
    l = _save_clip(d / "text_encoder", 16, 12, True)
    g = _save_clip(d / "text_encoder_2", 24, 16, True)
    t5 = _save_t5(d / "text_encoder_3", 64)
    for name, n in (("tokenizer", 77), ("tokenizer_2", 77), ("tokenizer_3", 256)):
        _tokenizer_dir(d / name, n)
    pipe = _load(d)
    from vllm_omni_b200.diffusion.models.sd3.pipeline import SD3PromptEncoder
    assert isinstance(pipe.text_encoder, SD3PromptEncoder)
    texts = ["a red cube on the table"]
    tok = transformers.AutoTokenizer.from_pretrained(str(d / "tokenizer"))
    tok3 = transformers.AutoTokenizer.from_pretrained(str(d / "tokenizer_3"))
    with torch.no_grad():
        ids = tok(texts, padding="max_length", max_length=77, truncation=True, return_tensors="pt").input_ids
        rl, rg = l(ids, output_hidden_states=True), g(ids, output_hidden_states=True)
        ids3 = tok3(texts, padding="max_length", max_length=40, truncation=True, return_tensors="pt").input_ids
        rt = t5(ids3).last_hidden_state
        clip = torch.nn.functional.pad(torch.cat([rl.hidden_states[-2], rg.hidden_states[-2]], -1), (0, 64 - 40))
        ref_pe, ref_pool = torch.cat([clip, rt], 1), torch.cat([rl.text_embeds, rg.text_embeds], -1)
        pe, mask = pipe.text_encoder(texts, "cpu", torch.float32, 40)
        pooled = pipe.pooled_encoder(texts, "cpu", torch.float32, 40)[0][:, 0]
    assert pe.shape == (1, 77 + 40, 64) and (pe - ref_pe).abs().max().item() < 2e-5 * max(1.0, ref_pe.abs().max().item())
    assert pooled.shape == (1, 28) and (pooled - ref_pool).abs().max().item() < 2e-5
    from vllm_omni_b200.diffusion.request import OmniDiffusionRequest
    from vllm_omni_b200.inputs import OmniDiffusionSamplingParams
    sp = OmniDiffusionSamplingParams(height=32, width=32, num_inference_steps=2, seed=1, output_type="latent", max_sequence_length=40,
                                     guidance_scale=4.0)
    out = pipe(OmniDiffusionRequest(prompts=[{"prompt": texts[0], "negative_prompt": "blurry"}], sampling_params=sp, request_ids=["r"]))
    assert torch.isfinite(out.output).all()


def test_wan_folder_attaches_umt5(tmp_path):
    import json
    pytest.importorskip("tokenizers")
    from vllm_omni_b200.diffusion.loader import DiffusersPipelineLoader
    from vllm_omni_b200.diffusion.models.text_encoders.t5 import T5PromptEncoder
    from vllm_omni_b200.entrypoints.omni_diffusion import build_diffusion_config
    torch.manual_seed(0)
    d = tmp_path
    (d / "model_index.json").write_text(json.dumps({"_class_name": "WanPipeline"}))
    (d / "transformer").mkdir()
    (d / "transformer" / "config.json").write_text(json.dumps(dict(_class_name="WanTransformer3DModel", num_attention_heads=2,
                                                                   attention_head_dim=24, text_dim=32, ffn_dim=64, num_layers=1)))
    hc = transformers.UMT5Config(vocab_size=40, d_model=32, d_kv=8, d_ff=64, num_layers=2, num_heads=2,
                                 relative_attention_num_buckets=8, relative_attention_max_distance=16, feed_forward_proj="gated-gelu")
    hf = _init(transformers.UMT5EncoderModel(hc))
    hf.save_pretrained(str(d / "text_encoder"))
    _tokenizer_dir(d / "tokenizer", 512)
    cfg = build_diffusion_config(str(d), dtype="float32", vae_config=dict(base_dim=8, num_res_blocks=1), output_type="latent")
    pipe = DiffusersPipelineLoader(cfg).load_model("cpu")
    assert isinstance(pipe.text_encoder, T5PromptEncoder) and pipe.text_encoder.model.cfg.per_layer_bias
    tok = transformers.AutoTokenizer.from_pretrained(str(d / "tokenizer"))
    enc = tok(["a red cube on the table"], padding="max_length", max_length=512, truncation=True, return_tensors="pt")
    with torch.no_grad():
        ref = hf(enc.input_ids, attention_mask=enc.attention_mask).last_hidden_state * enc.attention_mask[..., None]
        got = pipe._embeds(["a red cube on the table"], "prompt_embeds")
    assert got.shape == ref.shape and (got - ref).abs().max().item() < 2e-5 * max(1.0, ref.abs().max().item())
