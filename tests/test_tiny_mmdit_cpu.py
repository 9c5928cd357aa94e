"""BASELINE config 1: tiny MMDiT on CPU, fp32, seed 0, 4-step flow-match Euler, CFG 4.0."""
import torch

from vllm_omni_b200.entrypoints.omni import Omni
from vllm_omni_b200.inputs import OmniDiffusionSamplingParams


def _gen(omni, seed=0, steps=4, **kw):
    g = torch.Generator().manual_seed(1)
    pe, ne = torch.randn(32, 128, generator=g), torch.randn(32, 128, generator=g)
    sp = OmniDiffusionSamplingParams(height=256, width=256, num_inference_steps=steps, true_cfg_scale=4.0, seed=seed,
                                     **kw)
    return omni.generate([{"prompt": "", "negative_prompt": " ", "prompt_embeds": pe, "negative_prompt_embeds": ne}],
                         sp)


def test_tiny_mmdit_generates_deterministic_image():
    omni = Omni("TinyMMDiTPipeline", dtype="float32", device="cpu")
    try:
        a = _gen(omni)
        b = _gen(omni)
        c = _gen(omni, seed=1)
        assert a[0].images[0].size == (256, 256) and a[0].final_output_type == "image"
        ta, tb, tc = (torch.tensor(list(x[0].images[0].getdata())) for x in (a, b, c))
        assert torch.equal(ta, tb)
        assert not torch.equal(ta, tc)
    finally:
        omni.close()


def test_tiny_mmdit_latent_output_and_trajectory():
    omni = Omni("TinyMMDiTPipeline", dtype="float32", device="cpu", output_type="pt")
    try:
        r = _gen(omni, output_type="latent", return_trajectory_latents=True)
        assert r[0].latents is not None and r[0].latents.shape[0] == 4      # one snapshot per step
        assert torch.isfinite(r[0].latents).all()
    finally:
        omni.close()
