"""Every registered pipeline builds with a tiny geometry on CPU and produces output of the
right kind through the engine (image / video / audio)."""
import pytest
import torch

from vllm_omni_b200.diffusion.models.vae import autoencoder_kl_qwenimage as vq
from vllm_omni_b200.diffusion.registry import supported_models
from vllm_omni_b200.entrypoints.omni_diffusion import OmniDiffusion
from vllm_omni_b200.inputs import OmniDiffusionSamplingParams

FLUXY = dict(num_layers=1, num_single_layers=1, attention_head_dim=32, num_attention_heads=2, joint_attention_dim=32,
             pooled_projection_dim=16, in_channels=64, out_channels=16, axes_dims_rope=(8, 12, 12))
TINY = {
    "QwenImagePipeline": dict(num_layers=1, attention_head_dim=32, num_attention_heads=2, joint_attention_dim=32,
                              axes_dims_rope=(8, 12, 12)),
    "GlmImagePipeline": dict(num_layers=1, attention_head_dim=32, num_attention_heads=2, time_embed_dim=32, condition_dim=16,
                             prior_vq_quantizer_codebook_size=64, text_embed_dim=24, in_channels=16, out_channels=16),
    "TinyMMDiTPipeline": {},
    "FluxPipeline": FLUXY, "Flux2KleinPipeline": dict(FLUXY, out_channels=None, axes_dims_rope=(8, 8, 8, 8), timestep_guidance_channels=32), "LongCatImagePipeline": FLUXY, "LongCatImageEditPipeline": FLUXY,
    "OvisImagePipeline": FLUXY, "StableDiffusion3Pipeline": dict(FLUXY, num_single_layers=0),
    "ZImagePipeline": dict(dim=64, n_layers=1, n_refiner_layers=1, n_heads=2, n_kv_heads=2, cap_feat_dim=32,
                           axes_dims=(8, 12, 12), axes_lens=(128, 32, 32)),
    "BagelPipeline": dict(vocab_size=300, hidden_size=64, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1,
                          intermediate_size=64, max_latent_size=8, z_channels=16, start_of_image=290, end_of_image=291,
                          bos_token_id=288, eos_token_id=289),
    "WanPipeline": dict(num_attention_heads=2, attention_head_dim=24, text_dim=32, ffn_dim=64, num_layers=1),
    "WanImageToVideoPipeline": dict(num_attention_heads=2, attention_head_dim=24, text_dim=32, ffn_dim=64, num_layers=1),
    "Wan22TI2VPipeline": dict(num_attention_heads=2, attention_head_dim=24, text_dim=32, ffn_dim=64, num_layers=1),
    "HunyuanImage3Pipeline": dict(vocab_size=128, hidden_size=64, num_hidden_layers=1, num_attention_heads=2,
                                  num_key_value_heads=1, head_dim=32, num_experts=4, moe_topk=2, intermediate_size=32,
                                  moe_intermediate_size=32, patch_embed_hidden_dim=32, latent_channels=4),
    "StableAudioPipeline": dict(num_attention_heads=2, attention_head_dim=16, num_key_value_attention_heads=1, in_channels=8,
                                out_channels=8, cross_attention_dim=24, cross_attention_input_dim=24, global_states_input_dim=48,
                                time_proj_dim=16, num_layers=1, sample_size=6),
}


SMALL_KL = dict(block_out_channels=(8, 16, 16, 16), layers_per_block=1, norm_num_groups=4)   # read by the KL-VAE families


@pytest.fixture(autouse=True)
def small_vae(monkeypatch):
    orig = vq.QwenImageVAEConfig

    def tiny(*a, **k):
        k.setdefault("base_dim", 8)
        k.setdefault("num_res_blocks", 1)
        return orig(*a, **k)
    for mod in ("vllm_omni_b200.diffusion.models.qwen_image.pipeline",
                "vllm_omni_b200.diffusion.models.wan.pipeline"):
        import importlib
        m = importlib.import_module(mod)
        monkeypatch.setattr(m, "QwenImageVAEConfig", tiny)


@pytest.mark.parametrize("name", sorted(TINY))
def test_pipeline_runs_tiny(name):
    vae = SMALL_KL if name != "StableAudioPipeline" else dict(decoder_channels=8, channel_multiples=(1, 2),
                                                                downsampling_ratios=(2, 4), sampling_rate=800)
    if name == "HunyuanImage3Pipeline":                    # 1/16 fold-shuffle autoencoder: five levels
        vae = dict(block_out_channels=(8, 8, 8, 8, 8), layers_per_block=1, norm_num_groups=4)
    o = OmniDiffusion(name, dtype="float32", device="cpu", tf_model_config=TINY[name], vae_config=vae)
    try:
        sp = OmniDiffusionSamplingParams(height=64, width=64, num_inference_steps=2, seed=0, num_frames=5,
                                         guidance_scale=3.0, extra_args={"audio_seconds": 0.05})
        prompt = {"prompt": "a small test", "negative_prompt": " "}
        if name == "LongCatImageEditPipeline":             # an editing pipeline needs its input image
            from PIL import Image
            prompt["multi_modal_data"] = {"image": Image.new("RGB", (64, 64), (90, 120, 30))}
        out = o.generate([prompt], sp)[0]
        if name.startswith("Wan"):
            v = out.multimodal_output["video"]
            assert out.final_output_type == "video" and v.shape == (5, 64, 64, 3)
        elif name == "StableAudioPipeline":
            a = out.multimodal_output["audio"]
            assert out.final_output_type == "audio" and a.shape == (2, 40) and out.multimodal_output["sample_rate"] == 800
        else:
            assert out.images[0].size == (64, 64)
    finally:
        o.close()


def test_registry_lists_every_family_and_bagel_takes_injected_kv():
    names = supported_models()
    for n in ("QwenImagePipeline", "WanPipeline", "FluxPipeline", "ZImagePipeline", "StableDiffusion3Pipeline",
              "BagelPipeline", "HunyuanImage3Pipeline", "GlmImagePipeline", "LongCatImagePipeline", "OvisImagePipeline",
              "StableAudioPipeline", "Flux2KleinPipeline"):
        assert n in names
    o = OmniDiffusion("BagelPipeline", dtype="float32", device="cpu", tf_model_config=TINY["BagelPipeline"], vae_config=SMALL_KL)
    try:
        sp = OmniDiffusionSamplingParams(height=64, width=64, num_inference_steps=2, seed=0)
        sp.past_key_values = [(torch.randn(5, 1, 32), torch.randn(5, 1, 32))]          # the prompt context of an AR stage
        assert o.generate(["x"], sp)[0].images[0].size == (64, 64)
    finally:
        o.close()


def test_longcat_edit_appends_the_condition_image_as_a_second_frame():
    """LongCat-Image editing: the VAE latents of the input image follow the noise rows with modality
    id 2 on the first rotary axis; only the noise rows are stepped; the result depends on the image;
    a request without an image is refused."""
    import numpy as np
    from PIL import Image
    from vllm_omni_b200.diffusion.models.longcat_image.transformer import longcat_rope_angles
    a1 = longcat_rope_angles(2, 3, 4, (8, 12, 12), 16)
    a2 = longcat_rope_angles(2, 3, 4, (8, 12, 12), 16, frames=2)
    assert a2.shape[0] == 2 * 6 + 4
    assert torch.equal(a2[:6], a1[:6]) and torch.equal(a2[12:], a1[6:])
    assert torch.allclose(a2[6:12, 4:], a1[:6, 4:]) and not torch.allclose(a2[6:12, :4], a1[:6, :4])   # same (y, x), modality 2
    vae = dict(SMALL_KL)
    o = OmniDiffusion("LongCatImageEditPipeline", dtype="float32", device="cpu", tf_model_config=TINY["LongCatImageEditPipeline"],
                      vae_config=vae)
    try:
        sp = OmniDiffusionSamplingParams(height=64, width=64, num_inference_steps=2, seed=0, guidance_scale=3.0)
        rng = np.random.default_rng(0)
        imgs = [Image.fromarray(rng.integers(0, 255, (64, 64, 3), dtype=np.uint8)) for _ in range(2)]
        outs = [np.asarray(o.generate([{"prompt": "make it red", "negative_prompt": " ",
                                        "multi_modal_data": {"image": im}}], sp)[0].images[0], dtype=np.float32)
                for im in imgs]
        assert outs[0].shape == (64, 64, 3)
        assert np.abs(outs[0] - outs[1]).max() > 0          # the condition image reaches the network
        with pytest.raises(Exception):
            o.generate([{"prompt": "no image"}], sp)
    finally:
        o.close()


F64 = dict(num_layers=1, num_single_layers=1, attention_head_dim=64, num_attention_heads=2, joint_attention_dim=64,
           pooled_projection_dim=32, in_channels=64, out_channels=16, axes_dims_rope=(16, 24, 24))
GPU_CASES = {
    "WanPipeline": (dict(num_attention_heads=2, attention_head_dim=64, text_dim=64, ffn_dim=256, num_layers=1),
                    dict(base_dim=32, num_res_blocks=1)),
    "Flux2KleinPipeline": (dict(F64, out_channels=None, axes_dims_rope=(16, 16, 16, 16), timestep_guidance_channels=32), None),
    "StableDiffusion3Pipeline": (dict(F64, num_single_layers=0), None),
    "BagelPipeline": (dict(vocab_size=300, hidden_size=128, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1,
                           intermediate_size=128, max_latent_size=16, z_channels=16, start_of_image=290, end_of_image=291,
                           bos_token_id=288, eos_token_id=289), None),
    "GlmImagePipeline": (dict(num_layers=1, attention_head_dim=64, num_attention_heads=2, time_embed_dim=64, condition_dim=32,
                              prior_vq_quantizer_codebook_size=64, text_embed_dim=32, in_channels=16, out_channels=16), None),
    "LongCatImagePipeline": (F64, None),
    "OvisImagePipeline": (F64, None),
    "StableAudioPipeline": (dict(num_attention_heads=2, attention_head_dim=64, num_key_value_attention_heads=1, in_channels=8,
                                 out_channels=8, cross_attention_dim=32, cross_attention_input_dim=32, global_states_input_dim=64,
                                 time_proj_dim=16, num_layers=1, sample_size=6),
                            dict(decoder_channels=8, channel_multiples=(1, 2), downsampling_ratios=(2, 4), sampling_rate=800)),
}


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(GPU_CASES))
def test_pipeline_runs_on_a_gpu(name):
    """Kernel-friendly small geometries (head size 64) end to end on the device in bf16, VAE decode included (the
    channels-last GroupNorm and causal 3-D decoders run inside the pipelines)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    tf, vae = GPU_CASES[name]
    o = OmniDiffusion(name, dtype="bfloat16", device="cuda", tf_model_config=tf,
                      vae_config=vae if vae is not None else dict(block_out_channels=(32, 32, 32, 32), layers_per_block=1, norm_num_groups=8))
    try:
        sp = OmniDiffusionSamplingParams(height=128, width=128, num_inference_steps=2, seed=0, num_frames=5, guidance_scale=3.0,
                                         extra_args={"audio_seconds": 0.05})
        out = o.generate([{"prompt": "a small test", "negative_prompt": " "}], sp)[0]
        mm = out.multimodal_output or {}
        if "video" in mm:
            assert tuple(mm["video"].shape) == (5, 128, 128, 3)
        elif "audio" in mm:
            assert mm["audio"].shape[0] == 2 and torch.isfinite(torch.as_tensor(mm["audio"]).float()).all()
        else:
            assert out.images[0].size == (128, 128)
    finally:
        o.close()
