"""HunyuanImage-3: 2-D centred rotary positions, the prompt-K/V-cached two-launch attention against
a dense-mask oracle, checkpoint layouts (interleaved qkv, [up; gate] halves), the token-layout
patch embedders against NCHW PyTorch modules, the fold/unfold autoencoder, aspect buckets, and
tensor / CFG parallel runs against a single process (Gloo)."""
import math

import pytest
import torch
import torch.nn.functional as F
from torch import nn

from vllm_omni_b200.diffusion.models.hunyuan_image_3 import transformer as T
from vllm_omni_b200.diffusion.models.hunyuan_image_3.pipeline import HunyuanTokens, resolution_buckets, snap_resolution
from vllm_omni_b200.diffusion.models.vae import autoencoder_kl_conv3d as V

TINY = dict(vocab_size=128, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
            num_experts=4, moe_topk=2, intermediate_size=32, moe_intermediate_size=32, patch_embed_hidden_dim=32,
            latent_channels=4)


def test_rope2d_positions_centre_the_grid_on_its_diagonal_stretch():
    pos = T.rope2d_positions(5 + 6 + 2, 5, 2, 3)            # 5 text rows, a 2 x 3 grid, 2 rows after it
    assert pos[:5].tolist() == [[i, i] for i in range(5)]
    # by = 5 + (6 - 2) / 2 = 7, bx = 5 + (6 - 3) / 2 = 6.5 -> truncated after the column offset is added
    assert pos[5:11].tolist() == [[7, 6], [7, 7], [7, 8], [8, 6], [8, 7], [8, 8]]
    assert pos[11:].tolist() == [[11, 11], [12, 12]]
    cos, sin = T.rope2d_cos_sin(pos, 8, 10000.0)
    assert cos.shape == (13, 4)
    inv = [10000.0 ** (-2 * j / 8) for j in range(4)]
    y, x = 7.0, 8.0
    want = [math.cos(y * inv[0]), math.cos(x * inv[1]), math.cos(y * inv[2]), math.cos(x * inv[3])]
    assert torch.allclose(cos[7], torch.tensor(want), atol=1e-6)


def test_cached_steps_match_the_dense_mask_oracle():
    torch.manual_seed(0)
    cfg = T.HunyuanImage3Config.from_dict(TINY)
    m = T.HunyuanImage3Model(cfg, torch.float32, "cpu")
    for p in m.parameters():
        if p.dim() == 1:
            p.data.uniform_(0.5, 1.5)
    P, h, w = 5, 2, 3
    S = h * w
    cos, sin = T.rope2d_cos_sin(T.rope2d_positions(P + 1 + S, P + 1, h, w), cfg.head_dim)
    x0 = torch.randn(P + 1 + S, cfg.hidden_size)
    seqs = m.begin([P], S, "cpu")
    got0 = m(x0.clone(), seqs, cos, sin, first_step=True)
    want0 = T.reference_forward(m, x0, P, S, cos, sin)
    assert (got0 - want0).abs().max() < 2e-4
    # a later step: new <timestep> and image rows, the prompt's K/V come from the buffers
    tail = torch.randn(1 + S, cfg.hidden_size)
    got1 = m(tail.clone(), seqs, cos[P:], sin[P:], first_step=False)
    want1 = T.reference_forward(m, torch.cat([x0[:P], tail]), P, S, cos, sin)[P:]
    assert (got1 - want1).abs().max() < 2e-4
    # two sequences of different prompt length share the GEMMs
    P2 = 3
    c2, s2 = T.rope2d_cos_sin(T.rope2d_positions(P2 + 1 + S, P2 + 1, h, w), cfg.head_dim)
    xb = torch.randn(P2 + 1 + S, cfg.hidden_size)
    seqs2 = m.begin([P, P2], S, "cpu")
    both = m(torch.cat([x0, xb]), seqs2, torch.cat([cos, c2]), torch.cat([sin, s2]), first_step=True)
    assert (both[:P + 1 + S] - want0).abs().max() < 2e-4
    assert (both[P + 1 + S:] - T.reference_forward(m, xb, P2, S, c2, s2)).abs().max() < 2e-4


def test_checkpoint_layouts_interleaved_qkv_and_up_gate_halves():
    torch.manual_seed(1)
    cfg = T.HunyuanImage3Config.from_dict(dict(TINY, num_hidden_layers=1))
    m = T.HunyuanImage3Model(cfg, torch.float32, "cpu")
    H, Hkv, Dh, D = 4, 2, 16, 64
    q, k, v = torch.randn(H * Dh, D), torch.randn(Hkv * Dh, D), torch.randn(Hkv * Dh, D)
    G = H // Hkv
    inter = torch.cat([torch.cat([q.view(Hkv, G * Dh, D)[g], k.view(Hkv, Dh, D)[g], v.view(Hkv, Dh, D)[g]]) for g in range(Hkv)])
    gate, up = torch.randn(32, D), torch.randn(32, D)
    sd = [("model.layers.0.self_attn.qkv_proj.weight", inter),
          ("model.layers.0.mlp.experts.2.gate_and_up_proj.weight", torch.cat([up, gate])),
          ("model.layers.0.mlp.shared_mlp.gate_and_up_proj.weight", torch.cat([up, gate])),
          ("model.layers.0.mlp.gate.wg.weight", torch.randn(4, D)),
          ("model.layers.0.self_attn.query_layernorm.weight", torch.full((Dh,), 2.0)),
          ("model.wte.weight", torch.randn(128, D)), ("model.ln_f.weight", torch.ones(D))]
    loaded = m.load_weights(sd)
    assert len(loaded) == len(sd)
    L = m.layers[0]
    assert torch.equal(L.qkv_proj.weight.data, torch.cat([q, k, v]))
    assert torch.equal(L.w13.data[2], torch.cat([gate, up])) and torch.equal(L.shared_gate_up.weight.data, torch.cat([gate, up]))
    assert float(L.q_norm[0]) == 2.0


class _TorchResBlock(nn.Module):
    """NCHW restatement with stock modules (parameter names as in the checkpoint)."""

    def __init__(self, cin, emb, cout):
        super().__init__()
        self.in_layers = nn.Sequential(nn.GroupNorm(32, cin), nn.SiLU(), nn.Conv2d(cin, cout, 3, padding=1))
        self.emb_layers = nn.Sequential(nn.SiLU(), nn.Linear(emb, 2 * cout))
        self.out_layers = nn.Sequential(nn.GroupNorm(32, cout), nn.SiLU(), nn.Dropout(0.0), nn.Conv2d(cout, cout, 3, padding=1))
        self.skip_connection = nn.Conv2d(cin, cout, 1) if cin != cout else nn.Identity()

    def forward(self, x, emb):
        hh = self.in_layers(x)
        sc, sh = self.emb_layers(emb)[..., None, None].chunk(2, dim=1)
        hh = self.out_layers[1:](self.out_layers[0](hh) * (1 + sc) + sh)
        return self.skip_connection(x) + hh


def test_token_layout_resblock_matches_nchw_modules():
    torch.manual_seed(2)
    cin, emb, cout, h, w, B = 32, 48, 64, 3, 5, 2
    ref = _TorchResBlock(cin, emb, cout)
    for p in ref.parameters():
        p.data.normal_(0, 0.2)
    blk = T.ResBlock(cin, emb, cout, torch.float32, "cpu")
    missing = blk.load_state_dict(ref.state_dict(), strict=True)
    assert not missing.missing_keys
    x, e = torch.randn(B, cin, h, w), torch.randn(B, emb)
    want = ref(x, e).permute(0, 2, 3, 1).reshape(B, h * w, cout)
    got = blk(x.permute(0, 2, 3, 1).reshape(B, h * w, cin).contiguous(), e, h, w)
    assert (got - want).abs().max() < 2e-4
    # timestep embedder: cosines first, exact GELU
    te = T.TimestepEmbedder(64, torch.float32, "cpu")
    t = torch.tensor([0.0, 250.0, 999.0])
    sn = T.sinusoid(t, 256)
    assert torch.allclose(sn[0, :128], torch.ones(128)) and torch.allclose(sn[0, 128:], torch.zeros(128))
    want = F.linear(F.gelu(F.linear(sn, te.mlp[0].weight, te.mlp[0].bias)), te.mlp[2].weight, te.mlp[2].bias)
    assert torch.allclose(te(t), want, atol=1e-5)


def test_fold_unfold_autoencoder():
    x = torch.arange(2 * 3 * 2 * 4 * 6, dtype=torch.float32).view(2, 3, 2, 4, 6)
    for r1 in (1, 2):
        f = V._fold(x, r1)
        assert f.shape == (2, 3 * 4 * r1, 2 // r1, 2, 3)
        assert torch.equal(V._unfold(f, r1), x)
    # channel index is (r1, r2, r3, c): channel (0, 1, 0, c) holds the odd rows / even columns
    assert torch.equal(V._fold(x, 1)[:, 2 * 3:3 * 3], x[:, :, :, 1::2, 0::2])
    cfg = V.Conv3dVAEConfig(latent_channels=4, block_out_channels=(8, 8, 8, 8, 8), layers_per_block=1, norm_num_groups=4)
    vae = V.AutoencoderKLConv3D(cfg, with_encoder=True)
    img = torch.rand(1, 3, 32, 48) * 2 - 1
    z = vae.encode(img, sample=False)
    assert z.shape == (1, 4, 2, 3)
    out = vae.decode(z)
    assert out.shape == (1, 3, 32, 48) and torch.isfinite(out).all()
    # tiled decode covers the same canvas
    vae.use_tiling, vae.tile_latent = True, 2
    assert vae.decode(torch.randn(1, 4, 3, 5)).shape == (1, 3, 48, 80)
    # checkpoint names
    names = dict(vae.named_parameters())
    for n in ("decoder.up.0.block.0.conv1.weight", "decoder.up.0.upsample.conv.weight", "decoder.mid.attn_1.q.weight",
              "encoder.down.3.downsample.conv.weight", "decoder.conv_in.weight"):
        assert n in names, n
    assert "decoder.up.4.upsample.conv.weight" not in names


def test_resolution_buckets_and_special_tokens():
    b = resolution_buckets(1024)
    assert len(b) == 33 and b[16] == (1024, 1024) and b[0] == (512, 2048) and b[-1] == (2048, 512)
    assert snap_resolution(1024, 1024) == (1024, 1024, 16)
    hh, ww, i = snap_resolution(720, 1280)
    assert b[i] == (hh, ww) and abs(hh / ww - 720 / 1280) < 0.05
    tk = HunyuanTokens(128)
    cond, unc = tk.prompt_rows("a red cube", 16, uncond=False), tk.prompt_rows("a red cube", 16, uncond=True)
    assert len(cond) == len(unc) == 1 + 3 + 3
    assert unc[1:4] == [tk.cfg] * 3 and cond[-3:] == [tk.boi, tk.size_id, tk.ratio0 + 16] and cond[0] == tk.bos
    assert max(cond) < 128 and all(t < tk.n_text for t in cond[1:4])
    with pytest.raises(ValueError):
        HunyuanTokens(30)


def _run(par, scale=4.0):
    from vllm_omni_b200.entrypoints.omni import Omni
    from vllm_omni_b200.inputs import OmniDiffusionSamplingParams
    vae = dict(block_out_channels=(8, 8, 8, 8, 8), layers_per_block=1, norm_num_groups=4)
    omni = Omni("HunyuanImage3Pipeline", dtype="float32", device="cpu", tf_model_config=dict(TINY, num_key_value_heads=2),
                vae_config=vae, diffusion_load_format="dummy", parallel_config=par, output_type="latent")
    try:
        sp = OmniDiffusionSamplingParams(height=64, width=64, num_inference_steps=3, guidance_scale=scale, seed=0, output_type="latent")
        out = omni.generate([{"prompt": "a cube on a table"}], sp)[0]
        return torch.as_tensor(out.latents if out.latents is not None else out.images[0]).float()
    finally:
        omni.close()


def test_tensor_parallel_and_cfg_parallel_match_single_process():
    from vllm_omni_b200.diffusion.data import DiffusionParallelConfig
    a = _run(DiffusionParallelConfig())
    assert a.shape[-3:] == (4, 4, 4) and torch.isfinite(a).all()
    assert (a - _run(DiffusionParallelConfig(), scale=1.0)).abs().max() > 1e-6           # guidance reaches the result
    b = _run(DiffusionParallelConfig(tensor_parallel_size=2))
    assert (a - b).abs().max().item() < 1e-4
    c = _run(DiffusionParallelConfig(cfg_parallel_size=2))
    assert (a - c).abs().max().item() < 1e-4


@pytest.mark.gpu
def test_tiny_pipeline_runs_on_a_gpu():
    """The whole pipeline on the device kernels (two attention launches per layer against the kept prompt K/V, MoE
    chain, token-layout convolutions, fold / unfold autoencoder): a finite image of the requested size."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from vllm_omni_b200.entrypoints.omni import Omni
    from vllm_omni_b200.inputs import OmniDiffusionSamplingParams
    tf = dict(vocab_size=2048, hidden_size=512, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
              intermediate_size=512, moe_intermediate_size=256, num_experts=8, moe_topk=2, num_shared_expert=1,
              patch_embed_hidden_dim=128, latent_channels=32, vae_downsample=16, image_base_size=256,
              vae=dict(block_out_channels=(32, 64, 64, 128, 128), layers_per_block=1, norm_num_groups=8))
    o = Omni("HunyuanImage3Pipeline", dtype="bfloat16", device="cuda", tf_model_config=tf, diffusion_load_format="dummy",
             output_type="pt")
    try:
        sp = OmniDiffusionSamplingParams(height=256, width=256, num_inference_steps=3, guidance_scale=5.0, seed=0, output_type="pt")
        img = torch.as_tensor(o.generate([{"prompt": "a small red cube on a table"}], sp)[0].images[0]).float()
        assert tuple(img.shape) == (3, 256, 256) and torch.isfinite(img).all()
    finally:
        o.close()
