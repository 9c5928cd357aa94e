"""FLUX.2 transformer against a straight-line restatement of the published architecture on a dict of
diffusers-named tensors (joint sequence text-first, as published), the klein prompt encoder against
transformers' Qwen3 with padding, and the latent / schedule helpers."""
import math

import pytest
import torch
import torch.nn.functional as F

from vllm_omni_b200.diffusion.models.flux2.pipeline import compute_empirical_mu, patchify, unpatchify
from vllm_omni_b200.diffusion.models.flux2.transformer import (Flux2Transformer2DModel, Flux2TransformerConfig, image_ids,
                                                                 text_ids)

CFG = Flux2TransformerConfig(in_channels=16, num_layers=2, num_single_layers=2, attention_head_dim=16, num_attention_heads=3,
                             joint_attention_dim=40, timestep_guidance_channels=32, mlp_ratio=3.0, axes_dims_rope=(4, 4, 4, 4),
                             rope_theta=2000.0, guidance_embeds=True)


def rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def flux2_oracle(sd, c, hidden, enc, timestep, img_ids, txt_ids, guidance):
    D, H, Dh, eps = c.inner_dim, c.num_attention_heads, c.attention_head_dim, c.eps
    lin = lambda x, n: F.linear(x, sd[n + ".weight"])

    def sinus(t):
        half = c.timestep_guidance_channels // 2
        e = (t[:, None] * 1000.0) * torch.exp(-math.log(10000) * torch.arange(half) / half)[None]
        return torch.cat([e.cos(), e.sin()], -1)

    def mlp(x, pre):
        return lin(F.silu(lin(x, pre + ".linear_1")), pre + ".linear_2")
    temb = mlp(sinus(timestep), "time_guidance_embed.timestep_embedder") + mlp(sinus(guidance), "time_guidance_embed.guidance_embedder")

    def modulation(name, sets):
        m = lin(F.silu(temb), name + ".linear").unsqueeze(1).chunk(3 * sets, -1)
        return [m[3 * i:3 * i + 3] for i in range(sets)]
    mod_i, mod_t, mod_s = modulation("double_stream_modulation_img", 2), modulation("double_stream_modulation_txt", 2), \
        modulation("single_stream_modulation", 1)[0]
    x, ctx = lin(hidden, "x_embedder"), lin(enc, "context_embedder")

    def angles(ids):
        out = []
        for a, dim in enumerate(c.axes_dims_rope):
            inv = 1.0 / (c.rope_theta ** (torch.arange(0, dim, 2).double() / dim))
            out.append(ids[:, a].double()[:, None] * inv[None])
        return torch.cat(out, -1).float()
    ang = torch.cat([angles(txt_ids), angles(img_ids)], 0)              # text first
    cos, sin = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]

    def rope(t):                                                        # interleaved pairs
        a, b = t[..., 0::2], t[..., 1::2]
        return torch.stack([a * cos - b * sin, a * sin + b * cos], -1).flatten(-2)

    def attend(q, k, v):
        return F.scaled_dot_product_attention(rope(q).transpose(1, 2), rope(k).transpose(1, 2), v.transpose(1, 2)).transpose(1, 2).flatten(2)

    def swiglu(x):
        a, b = x.chunk(2, -1)
        return F.silu(a) * b
    B, St = ctx.shape[0], ctx.shape[1]
    ln = lambda t: F.layer_norm(t, (D,), eps=eps)
    for i in range(c.num_layers):
        p = f"transformer_blocks.{i}."
        (sh, sc, g), (sh2, sc2, g2) = mod_i
        (csh, csc, cg), (csh2, csc2, cg2) = mod_t
        nx, nc = (1 + sc) * ln(x) + sh, (1 + csc) * ln(ctx) + csh
        q, k, v = (lin(nx, p + f"attn.{n}").unflatten(-1, (H, Dh)) for n in ("to_q", "to_k", "to_v"))
        cq, ck, cv = (lin(nc, p + f"attn.{n}").unflatten(-1, (H, Dh)) for n in ("add_q_proj", "add_k_proj", "add_v_proj"))
        q, k = rms(q, sd[p + "attn.norm_q.weight"], eps), rms(k, sd[p + "attn.norm_k.weight"], eps)
        cq, ck = rms(cq, sd[p + "attn.norm_added_q.weight"], eps), rms(ck, sd[p + "attn.norm_added_k.weight"], eps)
        o = attend(torch.cat([cq, q], 1), torch.cat([ck, k], 1), torch.cat([cv, v], 1))
        co, o = o[:, :St], o[:, St:]
        x = x + g * lin(o, p + "attn.to_out.0")
        x = x + g2 * lin(swiglu(lin(ln(x) * (1 + sc2) + sh2, p + "ff.linear_in")), p + "ff.linear_out")
        ctx = ctx + cg * lin(co, p + "attn.to_add_out")
        ctx = ctx + cg2 * lin(swiglu(lin(ln(ctx) * (1 + csc2) + csh2, p + "ff_context.linear_in")), p + "ff_context.linear_out")
    h = torch.cat([ctx, x], 1)
    Fi = int(D * c.mlp_ratio)
    for i in range(c.num_single_layers):
        p = f"single_transformer_blocks.{i}."
        sh, sc, g = mod_s
        y = lin((1 + sc) * ln(h) + sh, p + "attn.to_qkv_mlp_proj")
        qkv, m = y.split([3 * D, 2 * Fi], -1)
        q, k, v = (t.unflatten(-1, (H, Dh)) for t in qkv.chunk(3, -1))
        q, k = rms(q, sd[p + "attn.norm_q.weight"], eps), rms(k, sd[p + "attn.norm_k.weight"], eps)
        h = h + g * lin(torch.cat([attend(q, k, v), swiglu(m)], -1), p + "attn.to_out")
    h = h[:, St:]
    scale, shift = lin(F.silu(temb), "norm_out.linear").chunk(2, -1)
    return lin(ln(h) * (1 + scale)[:, None] + shift[:, None], "proj_out")


def test_flux2_forward_from_diffusers_named_tensors():
    torch.manual_seed(0)
    m = Flux2Transformer2DModel(CFG, torch.float32, "cpu")
    params = dict(m.named_parameters())
    sd = {}
    for name, (pn, sl) in m.checkpoint_name_map().items():
        shape = list(params[pn].shape)
        if sl is not None:
            shape[0] = sl[1] - sl[0]
        sd[name] = torch.randn(shape) * 0.1 + (1.0 if ".norm_" in name else 0.0)
    assert m.load_weights(sd.items()) == set(sd)
    B, h, w, St = 2, 3, 4, 5
    hidden, enc = torch.randn(B, h * w, 16), torch.randn(B, St, 40)
    t, g = torch.tensor([0.7, 0.3]), torch.tensor([3.5, 1.0])
    ii, ti = image_ids(h, w), text_ids(St)
    ii = torch.cat([ii, image_ids(1, 2, t=10)])                          # plus two reference tokens at t = 10
    hidden = torch.cat([hidden, torch.randn(B, 2, 16)], 1)
    with torch.no_grad():
        out = m(hidden, enc, t, ii, ti, guidance=g)
        ref = flux2_oracle(sd, CFG, hidden, enc, t, ii, ti, g)
    assert out.shape == ref.shape == (B, h * w + 2, 16)
    assert (out - ref).abs().max().item() < 2e-4 * max(1.0, ref.abs().max().item())


def test_position_ids_and_latent_layout():
    ii = image_ids(2, 3, t=10)
    assert ii.tolist() == [[10, 0, 0, 0], [10, 0, 1, 0], [10, 0, 2, 0], [10, 1, 0, 0], [10, 1, 1, 0], [10, 1, 2, 0]]
    assert text_ids(3).tolist() == [[0, 0, 0, 0], [0, 0, 0, 1], [0, 0, 0, 2]]
    z = torch.randn(2, 3, 4, 6)
    p = patchify(z)
    assert p.shape == (2, 12, 2, 3) and torch.equal(unpatchify(p), z)
    assert torch.equal(p[0, 1 * 4 + 1 * 2 + 0, 1, 2], z[0, 1, 2 * 1 + 1, 2 * 2 + 0])     # channel (c, dy, dx)
    assert abs(compute_empirical_mu(4096, 50) - ((0.00016927 * 4096 + 0.45666666 - (8.73809524e-05 * 4096 + 1.89833333)) / 190 * 50
                                                 + (0.00016927 * 4096 + 0.45666666) - 200 * (0.00016927 * 4096 + 0.45666666 - (8.73809524e-05 * 4096 + 1.89833333)) / 190)) < 1e-9
    assert abs(compute_empirical_mu(5000, 4) - (0.00016927 * 5000 + 0.45666666)) < 1e-12


def test_klein_prompt_encoder_against_hf_qwen3_with_padding():
    transformers = pytest.importorskip("transformers")
    from vllm_omni_b200.diffusion.models.flux2.text_encoder import dense_hidden_states
    from vllm_omni_b200.models.qwen_decoder import DecoderConfig, QwenDecoderModel
    torch.manual_seed(1)
    hc = transformers.Qwen3Config(vocab_size=120, hidden_size=32, intermediate_size=64, num_hidden_layers=4, num_attention_heads=4,
                                  num_key_value_heads=2, head_dim=8, max_position_embeddings=128)
    hf = transformers.Qwen3ForCausalLM(hc).float().eval()
    m = QwenDecoderModel(DecoderConfig.from_dict(hc.to_dict()), torch.float32, "cpu", with_lm_head=False)
    m.load_weights([(n, w) for n, w in hf.state_dict().items() if not n.startswith("lm_head.")])
    ids = torch.randint(3, 120, (2, 12))
    mask = torch.ones(2, 12, dtype=torch.long)
    mask[0, 7:], mask[1, 10:] = 0, 0
    ids[0, 7:], ids[1, 10:] = 0, 0
    with torch.no_grad():
        r = hf(input_ids=ids, attention_mask=mask, output_hidden_states=True, use_cache=False).hidden_states
        mine = dense_hidden_states(m, ids, mask, (1, 2, 3))
    for k, got in zip((1, 2, 3), mine):
        assert (r[k] - got).abs().max().item() < 1e-4 * max(1.0, r[k].abs().max().item())     # padded rows included


def test_klein_pipeline_with_reference_image_and_bn_statistics():
    """Text-to-image and editing with a reference image at tiny geometry: the latent normalisation uses
    the autoencoder's batch-norm statistics from the checkpoint, reference rows are dropped from the
    output, and the edit result depends on the reference."""
    from vllm_omni_b200.diffusion.data import OmniDiffusionConfig, TransformerConfig
    from vllm_omni_b200.diffusion.models.flux2.pipeline import Flux2KleinPipeline
    from vllm_omni_b200.diffusion.request import OmniDiffusionRequest
    from vllm_omni_b200.inputs import OmniDiffusionSamplingParams
    torch.manual_seed(0)
    tf = dict(in_channels=16, num_layers=1, num_single_layers=1, attention_head_dim=16, num_attention_heads=2, joint_attention_dim=24,
              timestep_guidance_channels=32, axes_dims_rope=(4, 4, 4, 4), guidance_embeds=False)
    vae = dict(block_out_channels=(8, 16, 16, 16), layers_per_block=1, norm_num_groups=4)
    cfg = OmniDiffusionConfig(dtype=torch.float32, tf_model_config=TransformerConfig.from_dict(tf), vae_config=vae, output_type="latent")
    pipe = Flux2KleinPipeline(cfg, device="cpu")
    assert pipe.vae.cfg.latent_channels == 4 and pipe.vae.post_quant_conv is not None and pipe.vae.cfg.scaling_factor == 1.0
    mean, var = torch.randn(16), torch.rand(16) + 0.5
    assert pipe.load_weights([("vae.bn.running_mean", mean), ("vae.bn.running_var", var)]) == {"vae.bn.running_mean", "vae.bn.running_var"}
    sp = lambda: OmniDiffusionSamplingParams(height=64, width=64, num_inference_steps=2, seed=3, output_type="latent", max_sequence_length=8)
    run = lambda prompt: pipe(OmniDiffusionRequest(prompts=[prompt], sampling_params=sp(), request_ids=["r"])).output
    base = run("a cube")
    assert base.shape == (1, 4, 8, 8) and torch.isfinite(base).all()
    img = torch.rand(3, 48, 64) * 2 - 1
    a = run({"prompt": "a cube", "multi_modal_data": {"image_tensor": [img]}})
    b = run({"prompt": "a cube", "multi_modal_data": {"image_tensor": [-img]}})
    assert a.shape == base.shape and not torch.allclose(a, base) and not torch.allclose(a, b)
    # de-normalisation: zero velocity would leave noise * std + mean; check the affine map on a known tensor
    m, s = pipe._bn()
    assert torch.allclose(m.flatten(), mean) and torch.allclose(s.flatten(), torch.sqrt(var + pipe.bn_eps))
