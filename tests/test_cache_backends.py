"""TeaCache / DBCache on the tiny pipeline (CPU): thresholds 0 reproduce the uncached image,
large thresholds skip blocks and stay close."""
import torch

from vllm_omni_b200.entrypoints.omni_diffusion import OmniDiffusion
from vllm_omni_b200.inputs import OmniDiffusionSamplingParams


def _run(**kw):
    o = OmniDiffusion("TinyMMDiTPipeline", dtype="float32", device="cpu", output_type="pt", **kw)
    try:
        sp = OmniDiffusionSamplingParams(height=128, width=128, num_inference_steps=8, true_cfg_scale=3.0, seed=3,
                                         output_type="latent")
        out = o.generate([{"prompt": "a red fox", "negative_prompt": " "}], sp)
        runner = o.engine.executor.worker.model_runner
        stats = runner.cache_backend.summary() if runner.cache_backend else None
        return out[0].images[0] if out[0].images else None, stats, out
    finally:
        o.close()


def _latent(out):
    # latent output: post-processing passes the packed latents through unchanged
    return out[2][0].images[0] if out[2][0].images else out[2][0].latents


def test_teacache_zero_threshold_is_exact_and_large_threshold_skips():
    base = _run()
    exact = _run(cache_backend="tea_cache", cache_config={"rel_l1_thresh": 0.0, "coefficients": [0, 0, 0, 1.0, 0]})
    assert exact[1]["skipped_steps"] == 0
    assert torch.allclose(_latent(base), _latent(exact), atol=1e-5)
    fast = _run(cache_backend="tea_cache", cache_config={"rel_l1_thresh": 1e9, "coefficients": [0, 0, 0, 1.0, 0]})
    assert fast[1]["skipped_steps"] >= 4 and fast[1]["steps"] == 8
    assert torch.isfinite(_latent(fast)).all()


def test_dbcache_thresholds_and_taylorseer():
    base = _run()
    exact = _run(cache_backend="cache_dit", cache_config={"residual_diff_threshold": 0.0, "max_warmup_steps": 0})
    assert exact[1]["skipped_steps"] == 0
    assert torch.allclose(_latent(base), _latent(exact), atol=1e-5)
    fast = _run(cache_backend="cache_dit", cache_config={"residual_diff_threshold": 1e9, "max_warmup_steps": 2,
                                                         "max_continuous_cached_steps": 2, "enable_taylorseer": True})
    assert 2 <= fast[1]["skipped_steps"] <= 5 and fast[1]["block_skip_ratio"] > 0
    assert torch.isfinite(_latent(fast)).all()


# ----------------------------------------------------------------------------- the other model families
def _zoo(name, **kw):
    from test_model_zoo import SMALL_KL, TINY
    import importlib
    import vllm_omni_b200.diffusion.models.vae.autoencoder_kl_qwenimage as vq
    orig = vq.QwenImageVAEConfig
    mods = [importlib.import_module(m) for m in ("vllm_omni_b200.diffusion.models.qwen_image.pipeline",
                                                 "vllm_omni_b200.diffusion.models.wan.pipeline")]
    tiny = lambda *a, **k: orig(*a, **{**dict(base_dim=8, num_res_blocks=1), **k})
    for m in mods:
        m.QwenImageVAEConfig = tiny
    tf = dict(TINY[name])
    for k in ("num_layers", "num_single_layers", "n_layers", "num_hidden_layers"):
        if k in tf:
            tf[k] = 3                                         # enough blocks for first / middle / last groups
    try:
        o = OmniDiffusion(name, dtype="float32", device="cpu", tf_model_config=tf, vae_config=SMALL_KL, output_type="latent", **kw)
        try:
            sp = OmniDiffusionSamplingParams(height=64, width=64, num_inference_steps=6, seed=0, num_frames=5, guidance_scale=3.0,
                                             output_type="latent")
            out = o.generate([{"prompt": "a small test", "negative_prompt": " "}], sp)[0]
            runner = o.engine.executor.worker.model_runner
            stats = runner.cache_backend.summary() if runner.cache_backend else None
            lat = out.latents if out.latents is not None else (out.images[0] if out.images else out.multimodal_output.get("video"))
            return torch.as_tensor(lat).float(), stats
        finally:
            o.close()
    finally:
        for m in mods:
            m.QwenImageVAEConfig = orig


import pytest


@pytest.mark.parametrize("name", ["FluxPipeline", "StableDiffusion3Pipeline", "Flux2KleinPipeline", "ZImagePipeline", "WanPipeline",
                                  "BagelPipeline", "LongCatImagePipeline", "OvisImagePipeline"])
def test_cache_backends_on_every_family_with_a_block_stack(name):
    """Thresholds of zero reproduce the uncached sample exactly; permissive thresholds skip work.  Pipelines
    that evaluate the guidance branches in separate calls (FLUX.2-klein, BAGEL) keep one state per branch."""
    base, _ = _zoo(name)
    tea0, s = _zoo(name, cache_backend="tea_cache", cache_config={"rel_l1_thresh": 0.0, "coefficients": [0, 0, 0, 1.0, 0]})
    assert s["skipped_steps"] == 0 and s["steps"] >= 5 and torch.allclose(base, tea0, atol=1e-5)
    tea, s = _zoo(name, cache_backend="tea_cache", cache_config={"rel_l1_thresh": 1e9, "coefficients": [0, 0, 0, 1.0, 0]})
    assert s["skipped_steps"] >= 2 and torch.isfinite(tea).all()
    db0, s = _zoo(name, cache_backend="cache_dit", cache_config={"residual_diff_threshold": 0.0, "max_warmup_steps": 0})
    assert s["skipped_steps"] == 0 and torch.allclose(base, db0, atol=1e-5)
    db, s = _zoo(name, cache_backend="cache_dit", cache_config={"residual_diff_threshold": 1e9, "max_warmup_steps": 1,
                                                                "max_continuous_cached_steps": 2, "enable_taylorseer": True,
                                                                "Fn_compute_blocks": 1, "Bn_compute_blocks": 1})
    assert s["skipped_steps"] >= 1 and s["block_skip_ratio"] > 0 and torch.isfinite(db).all()


def test_teacache_accumulates_absolute_rescaled_distance_like_the_reference_loop():
    """Coefficients whose polynomial is negative at small rel (the Qwen-Image set ends in -2.0e-02):
    the accumulator adds |poly(rel)| as the reference hook does (teacache/hook.py:225), so the skip
    sequence equals a straight restatement of that loop."""
    import numpy as np
    from vllm_omni_b200.ops.fused import RelL1State, rel_l1_update
    coef = [-4.50000000e+02, 2.80000000e+02, -4.50000000e+01, 3.20000000e+00, -2.00000000e-02]
    thresh = 0.06
    torch.manual_seed(0)
    base = torch.randn(4, 64, 32)
    rels = [0.001, 0.002, 0.004, 0.05, 0.003, 0.001, 0.08, 0.002, 0.002, 0.002, 0.03]
    st = RelL1State("cpu", coef, thresh)
    acc, want, got = 0.0, [], []
    poly = np.poly1d(coef)
    prev = base
    for r in rels:
        cur = prev + r * prev.abs().mean() / 0.7979 * torch.randn_like(prev)      # E|N(0,1)| = 0.7979
        rel = float(((cur - prev).abs().mean() / (prev.abs().mean() + 1e-8)))
        acc += abs(float(poly(rel)))
        if acc < thresh:
            want.append(1)
        else:
            want.append(0)
            acc = 0.0
        rel_l1_update(cur, prev, st)
        got.append(int(st.state[2]))
        prev = cur
    assert got == want
    assert 0 < sum(want) < len(want)
