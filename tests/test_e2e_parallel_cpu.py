"""End-to-end equivalence through the public API: ``Omni`` with a parallel configuration (two CPU
worker processes over Gloo, spawned by the multi-process executor) produces the image of the
single-process run.  Tiny random-weight Qwen-Image geometry, 128 x 128, 2 steps, true CFG."""
import pytest
import torch

from vllm_omni_b200.diffusion.data import DiffusionParallelConfig
from vllm_omni_b200.entrypoints.omni import Omni
from vllm_omni_b200.inputs import OmniDiffusionSamplingParams

TC = dict(num_layers=2, attention_head_dim=32, num_attention_heads=4, joint_attention_dim=64, axes_dims_rope=(8, 12, 12))


def _image(par: DiffusionParallelConfig) -> torch.Tensor:
    omni = Omni("QwenImagePipeline", dtype="float32", device="cpu", tf_model_config=TC, diffusion_load_format="dummy",
                parallel_config=par, output_type="pt")
    try:
        g = torch.Generator().manual_seed(1)
        pe, ne = torch.randn(8, 64, generator=g), torch.randn(8, 64, generator=g)
        sp = OmniDiffusionSamplingParams(height=128, width=128, num_inference_steps=2, true_cfg_scale=4.0, seed=0,
                                         output_type="pt")
        out = omni.generate([{"prompt": "", "negative_prompt": " ", "prompt_embeds": pe, "negative_prompt_embeds": ne}], sp)
        return torch.as_tensor(out[0].images[0]).float()
    finally:
        omni.close()


@pytest.fixture(scope="module")
def baseline():
    return _image(DiffusionParallelConfig())


@pytest.mark.parametrize("kw", [dict(ulysses_degree=2), dict(ring_degree=2), dict(cfg_parallel_size=2),
                                dict(tensor_parallel_size=2)], ids=["ulysses2", "ring2", "cfg2", "tp2"])
def test_parallel_config_matches_single_process(baseline, kw):
    img = _image(DiffusionParallelConfig(**kw))
    assert img.shape == baseline.shape
    d = (img - baseline).abs()
    assert d.mean().item() < 2e-4 and d.max().item() < 2e-3, (d.mean().item(), d.max().item())


def test_flux2_klein_cfg_parallel_matches_single_process():
    """FLUX.2-klein under classifier-free guidance: one guidance branch per rank equals both on one rank."""
    tf = dict(in_channels=64, num_layers=1, num_single_layers=1, attention_head_dim=32, num_attention_heads=2,
              joint_attention_dim=32, timestep_guidance_channels=32, axes_dims_rope=(8, 8, 8, 8), guidance_embeds=False)
    vae = dict(block_out_channels=(8, 16, 16, 16), layers_per_block=1, norm_num_groups=4)

    def run(par):
        omni = Omni("Flux2KleinPipeline", dtype="float32", device="cpu", tf_model_config=tf, vae_config=vae,
                    diffusion_load_format="dummy", parallel_config=par, output_type="latent")
        try:
            sp = OmniDiffusionSamplingParams(height=64, width=64, num_inference_steps=3, guidance_scale=4.0, seed=0,
                                             output_type="latent", max_sequence_length=8)
            out = omni.generate(["a cube"], sp)[0]
            return torch.as_tensor(out.latents if out.latents is not None else out.images[0]).float()
        finally:
            omni.close()
    a, b = run(DiffusionParallelConfig()), run(DiffusionParallelConfig(cfg_parallel_size=2))
    assert a.shape == b.shape and (a - b).abs().max().item() < 1e-4


@pytest.mark.parametrize("name", ["LongCatImagePipeline", "OvisImagePipeline", "StableDiffusion3Pipeline"])
def test_true_cfg_families_match_under_cfg_parallel(name):
    """LongCat-Image (guided velocity clamped per token) and Ovis-Image run true guidance against the negative
    prompt; with one branch per rank the latents equal the single-process run, and guidance changes them."""
    tf = dict(num_layers=1, num_single_layers=1, attention_head_dim=32, num_attention_heads=2, joint_attention_dim=32,
              pooled_projection_dim=16, in_channels=64, out_channels=16, axes_dims_rope=(8, 12, 12))
    if name == "StableDiffusion3Pipeline":
        tf = dict(tf, num_single_layers=0, num_layers=2)
    vae = dict(block_out_channels=(8, 16, 16, 16), layers_per_block=1, norm_num_groups=4)

    def run(par, scale):
        omni = Omni(name, dtype="float32", device="cpu", tf_model_config=tf, vae_config=vae, diffusion_load_format="dummy",
                    parallel_config=par, output_type="latent")
        try:
            sp = OmniDiffusionSamplingParams(height=64, width=64, num_inference_steps=3, guidance_scale=scale, seed=0,
                                             output_type="latent", max_sequence_length=8)
            out = omni.generate([{"prompt": "a cube", "negative_prompt": "blurry"}], sp)[0]
            return torch.as_tensor(out.latents if out.latents is not None else out.images[0]).float()
        finally:
            omni.close()
    a, b = run(DiffusionParallelConfig(), 4.0), run(DiffusionParallelConfig(cfg_parallel_size=2), 4.0)
    assert a.shape == b.shape and (a - b).abs().max().item() < 1e-4
    assert (a - run(DiffusionParallelConfig(), 1.0)).abs().max().item() > 1e-6


def test_wan_cfg_parallel_matches_single_process():
    """Wan text-to-video: the UniPC step runs on both ranks from the gathered branch velocities."""
    tf = dict(num_attention_heads=2, attention_head_dim=24, text_dim=32, ffn_dim=64, num_layers=1)

    def run(par):
        omni = Omni("WanPipeline", dtype="float32", device="cpu", tf_model_config=tf, vae_config=dict(base_dim=8, num_res_blocks=1),
                    diffusion_load_format="dummy", parallel_config=par, output_type="latent")
        try:
            sp = OmniDiffusionSamplingParams(height=32, width=32, num_frames=5, num_inference_steps=3, guidance_scale=4.0, seed=0,
                                             output_type="latent")
            out = omni.generate([{"prompt": "a cube", "negative_prompt": "blurry"}], sp)[0]
            lat = out.latents if out.latents is not None else out.multimodal_output.get("video")
            return torch.as_tensor(lat).float()
        finally:
            omni.close()
    a, b = run(DiffusionParallelConfig()), run(DiffusionParallelConfig(cfg_parallel_size=2))
    assert a.shape == b.shape and (a - b).abs().max().item() < 1e-4


def test_flux_tensor_parallel_matches_single_process():
    """FLUX (double-stream + single-stream blocks) with heads and MLP columns split over two ranks."""
    tf = dict(num_layers=1, num_single_layers=2, attention_head_dim=32, num_attention_heads=2, joint_attention_dim=32,
              pooled_projection_dim=16, in_channels=64, out_channels=16, axes_dims_rope=(8, 12, 12))
    vae = dict(block_out_channels=(8, 16, 16, 16), layers_per_block=1, norm_num_groups=4)

    def run(par):
        omni = Omni("FluxPipeline", dtype="float32", device="cpu", tf_model_config=tf, vae_config=vae,
                    diffusion_load_format="dummy", parallel_config=par, output_type="latent")
        try:
            sp = OmniDiffusionSamplingParams(height=64, width=64, num_inference_steps=3, guidance_scale=3.5, seed=0,
                                             output_type="latent", max_sequence_length=8)
            out = omni.generate(["a cube"], sp)[0]
            return torch.as_tensor(out.latents if out.latents is not None else out.images[0]).float()
        finally:
            omni.close()
    a, b = run(DiffusionParallelConfig()), run(DiffusionParallelConfig(tensor_parallel_size=2))
    assert a.shape == b.shape and (a - b).abs().max().item() < 1e-4


def test_wan_tensor_parallel_matches_single_process():
    """Wan with heads / FFN columns over two ranks; the q / k RMSNorms span all heads, so their mean
    squares are summed across the ranks."""
    tf = dict(num_attention_heads=2, attention_head_dim=24, text_dim=32, ffn_dim=64, num_layers=2)

    def run(par):
        omni = Omni("WanPipeline", dtype="float32", device="cpu", tf_model_config=tf, vae_config=dict(base_dim=8, num_res_blocks=1),
                    diffusion_load_format="dummy", parallel_config=par, output_type="latent")
        try:
            sp = OmniDiffusionSamplingParams(height=32, width=32, num_frames=5, num_inference_steps=2, guidance_scale=3.0, seed=0,
                                             output_type="latent")
            out = omni.generate([{"prompt": "a cube", "negative_prompt": "blurry"}], sp)[0]
            lat = out.latents if out.latents is not None else out.multimodal_output.get("video")
            return torch.as_tensor(lat).float()
        finally:
            omni.close()
    a, b = run(DiffusionParallelConfig()), run(DiffusionParallelConfig(tensor_parallel_size=2))
    assert a.shape == b.shape and (a - b).abs().max().item() < 1e-4


def test_z_image_ulysses_matches_single_process():
    """Z-Image (single stream, unified [image | caption] rows sharded over the group) through ``Omni``."""
    tf = dict(dim=64, n_layers=1, n_refiner_layers=1, n_heads=2, n_kv_heads=2, cap_feat_dim=32, axes_dims=(8, 12, 12),
              axes_lens=(128, 32, 32))
    vae = dict(block_out_channels=(8, 16, 16, 16), layers_per_block=1, norm_num_groups=4)

    def run(par):
        omni = Omni("ZImagePipeline", dtype="float32", device="cpu", tf_model_config=tf, vae_config=vae,
                    diffusion_load_format="dummy", parallel_config=par, output_type="latent")
        try:
            sp = OmniDiffusionSamplingParams(height=64, width=64, num_inference_steps=2, guidance_scale=3.5, seed=0,
                                             output_type="latent", max_sequence_length=8)
            out = omni.generate([{"prompt": "a cube", "negative_prompt": "blurry"}], sp)[0]
            return torch.as_tensor(out.latents if out.latents is not None else out.images[0]).float()
        finally:
            omni.close()
    a, b = run(DiffusionParallelConfig()), run(DiffusionParallelConfig(ulysses_degree=2))
    assert a.shape == b.shape and (a - b).abs().max().item() < 1e-4
