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
