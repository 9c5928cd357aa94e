"""End-to-end equivalence on two GPUs through the public API: ``Omni`` with a parallel configuration (two
worker processes over NCCL, the sm_100a kernels and their fused exchanges underneath) against the
single-GPU run of the same random-weight model.  bf16, head sizes the tcgen05 attention covers (64 / 128);
the tolerances are those of two bf16 runs that sum in a different order."""
import pytest
import torch

from vllm_omni_b200.diffusion.data import DiffusionParallelConfig
from vllm_omni_b200.entrypoints.omni import Omni
from vllm_omni_b200.inputs import OmniDiffusionSamplingParams

pytestmark = pytest.mark.gpu

VAE_KL = dict(block_out_channels=(32, 32, 32, 32), layers_per_block=1, norm_num_groups=8)
CASES = {
    # name -> (pipeline, transformer config, vae config, sampling kwargs)
    "flux": ("FluxPipeline",
             dict(num_layers=2, num_single_layers=2, attention_head_dim=64, num_attention_heads=4, joint_attention_dim=64,
                  pooled_projection_dim=32, in_channels=64, out_channels=16, axes_dims_rope=(16, 24, 24)),
             VAE_KL, dict(height=256, width=256, guidance_scale=3.5, max_sequence_length=16)),
    "wan": ("WanPipeline",
            dict(num_attention_heads=4, attention_head_dim=64, text_dim=64, ffn_dim=512, num_layers=2),
            dict(base_dim=8, num_res_blocks=1), dict(height=128, width=128, num_frames=9, guidance_scale=3.0)),
    "z_image": ("ZImagePipeline",
                dict(dim=384, n_layers=2, n_refiner_layers=1, n_heads=6, n_kv_heads=6, cap_feat_dim=32,
                     axes_dims=(16, 24, 24), axes_lens=(256, 64, 64)),
                VAE_KL, dict(height=256, width=256, guidance_scale=3.5, max_sequence_length=16)),
}


def _need_two():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")


def _latents(case: str, par: DiffusionParallelConfig) -> torch.Tensor:
    name, tf, vae, kw = CASES[case]
    omni = Omni(name, dtype="bfloat16", device="cuda", tf_model_config=tf, vae_config=vae, diffusion_load_format="dummy",
                parallel_config=par, output_type="latent")
    try:
        sp = OmniDiffusionSamplingParams(num_inference_steps=3, seed=0, output_type="latent", **kw)
        out = omni.generate([{"prompt": "a cube", "negative_prompt": "blurry"}], sp)[0]
        lat = out.latents if out.latents is not None else (out.images[0] if out.images else out.multimodal_output.get("video"))
        return torch.as_tensor(lat).float().cpu()
    finally:
        omni.close()


_single: dict[str, torch.Tensor] = {}


def _check(case: str, par: DiffusionParallelConfig):
    _need_two()
    if case not in _single:
        _single[case] = _latents(case, DiffusionParallelConfig())
    a, b = _single[case], _latents(case, par)
    assert a.shape == b.shape and torch.isfinite(b).all()
    d = (a - b).abs()
    scale = a.abs().mean().item() + 1e-6
    assert d.mean().item() < 0.03 * scale + 2e-3 and d.max().item() < 0.5 * scale + 0.05, (d.mean().item(), d.max().item(), scale)


@pytest.mark.parametrize("case", ["flux", "wan"])
def test_tensor_parallel_two_gpus(case):
    _check(case, DiffusionParallelConfig(tensor_parallel_size=2))


@pytest.mark.parametrize("case", ["wan", "z_image"])
def test_ulysses_two_gpus(case):
    _check(case, DiffusionParallelConfig(ulysses_degree=2))


def test_wan_ring_two_gpus():
    _check("wan", DiffusionParallelConfig(ring_degree=2))


def test_flux_cfg_parallel_is_refused_or_matches():
    """FLUX uses distilled guidance (one branch): a CFG-parallel request either runs as one branch per rank
    with equal results or is refused with a message; it must not hang or return garbage."""
    _need_two()
    try:
        _check("flux", DiffusionParallelConfig(cfg_parallel_size=2))
    except (ValueError, RuntimeError, NotImplementedError) as e:
        assert "cfg" in str(e).lower() or "guidance" in str(e).lower()


def test_fp8_pipeline_one_gpu_close_to_bf16():
    """``quantization="fp8"`` through the public API on a GPU: the block-scaled e4m3 GEMM kernel carries the
    eligible linear layers; the latents stay close to the bf16 run and are not identical to it."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    tf = dict(num_layers=2, num_single_layers=2, attention_head_dim=128, num_attention_heads=2, joint_attention_dim=128,
              pooled_projection_dim=32, in_channels=64, out_channels=16, axes_dims_rope=(32, 48, 48))

    def run(**kw):
        omni = Omni("FluxPipeline", dtype="bfloat16", device="cuda", tf_model_config=tf, vae_config=VAE_KL,
                    diffusion_load_format="dummy", output_type="latent", **kw)
        try:
            sp = OmniDiffusionSamplingParams(num_inference_steps=3, seed=0, output_type="latent", height=256, width=256,
                                             guidance_scale=3.5, max_sequence_length=16)
            out = omni.generate(["a cube"], sp)[0]
            return torch.as_tensor(out.latents if out.latents is not None else out.images[0]).float().cpu()
        finally:
            omni.close()
    a = run()
    b = run(quantization="fp8", quantization_config={"min_features": 128})
    assert a.shape == b.shape and torch.isfinite(b).all()
    rel = ((a - b).norm() / a.norm()).item()
    assert 0.0 < rel < 0.15, rel
