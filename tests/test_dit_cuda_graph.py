"""Generic CUDA-graph replay of a denoiser forward (models without a captured loop of their own)."""
import pytest
import torch

from vllm_omni_b200.diffusion.graphed import GraphedForward, _sig


def test_signature_and_cpu_passthrough():
    calls = []

    def f(x, n, flags=(1, 2), opt=None):
        calls.append(n)
        return x * n
    g = GraphedForward(f)
    x = torch.ones(3)
    assert torch.equal(g(x, 2), x * 2) and torch.equal(g(x, 3, flags=[4]), x * 3) and calls == [2, 3]
    assert g.replays == 0 and not g.entries                      # CPU tensors never enter the graph path
    # host tensors count by value (position ids and the like), device tensors by layout
    assert _sig((x, 1, None, "a", [1.5, (2,)])) == _sig((torch.ones(3), 1, None, "a", [1.5, (2,)]))
    assert _sig((x,)) != _sig((torch.zeros(3),)) and _sig((x,)) != _sig((torch.ones(4),))
    with pytest.raises(TypeError):
        _sig(object())
    assert torch.equal(g(x, 2), x * 2)


def _replay_vs_eager(monkeypatch, name, tf, prompt_len):
    from vllm_omni_b200.diffusion import graphed as G
    from vllm_omni_b200.entrypoints.omni import Omni
    from vllm_omni_b200.inputs import OmniDiffusionSamplingParams
    vae = dict(block_out_channels=(32, 32, 32, 32), layers_per_block=1, norm_num_groups=8)

    def run(flag):
        monkeypatch.setenv("OMNI_DIT_CUDA_GRAPH", flag)
        omni = Omni(name, dtype="bfloat16", device="cuda", tf_model_config=tf, vae_config=vae,
                    diffusion_load_format="dummy", output_type="latent")
        try:
            sp = OmniDiffusionSamplingParams(height=128, width=128, num_inference_steps=5, guidance_scale=3.5, seed=0,
                                             output_type="latent", max_sequence_length=prompt_len)
            out = omni.generate(["a cube"], sp)[0]
            return torch.as_tensor(out.latents if out.latents is not None else out.images[0]).float().cpu()
        finally:
            omni.close()
    before = G.total_replays
    eager = run("0")
    assert G.total_replays == before
    graphed = run("1")
    assert G.total_replays - before >= 3            # 5 steps: one eager, one capture + replay, three replays
    assert eager.shape == graphed.shape and torch.isfinite(graphed).all()
    assert (eager - graphed).abs().max().item() < 1e-3


@pytest.mark.gpu
def test_flux_forward_replayed_from_a_graph_equals_eager(monkeypatch):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    tf = dict(num_layers=1, num_single_layers=2, attention_head_dim=64, num_attention_heads=2, joint_attention_dim=64,
              pooled_projection_dim=32, in_channels=64, out_channels=16, axes_dims_rope=(16, 24, 24))
    _replay_vs_eager(monkeypatch, "FluxPipeline", tf, 16)


@pytest.mark.gpu
def test_z_image_forward_replayed_from_a_graph_equals_eager(monkeypatch):
    """Its position tables, pad-row masks and key lengths come from the per-geometry layout cache, so the
    captured call copies nothing from the host."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    tf = dict(dim=192, n_layers=1, n_refiner_layers=1, n_heads=3, n_kv_heads=3, cap_feat_dim=32,     # MLP width 512
              axes_dims=(16, 24, 24), axes_lens=(128, 32, 32))
    _replay_vs_eager(monkeypatch, "ZImagePipeline", tf, 16)
