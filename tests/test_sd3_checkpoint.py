"""SD3 MMDiT against a straight-line PyTorch restatement of the published architecture on a dict of
diffusers-named tensors: conv patch embedding + cropped sin/cos table, joint attention without
rotary embedding, AdaLN-Zero blocks, ``context_pre_only`` last block, AdaLN-continuous output."""
import math

import numpy as np
import torch
import torch.nn.functional as F

from vllm_omni_b200.diffusion.models.qwen_image.pipeline import pack_latents
from vllm_omni_b200.diffusion.models.sd3.transformer import SD3Transformer2DModel, SD3TransformerConfig


def _sinus(t):
    half = 128
    e = (t.float()[:, None] * 1000.0) * torch.exp(-math.log(10000.0) * torch.arange(half).float() / half)[None]
    return torch.cat([e.cos(), e.sin()], -1)


def _pos_table(dim, grid, base):
    """numpy restatement of the 2-D sin/cos table (x coordinate in the first half)."""
    gh = np.arange(grid, dtype=np.float64) / (grid / base)
    gw = np.arange(grid, dtype=np.float64) / (grid / base)
    X, Y = np.meshgrid(gw, gh)
    def one(d, pos):
        om = 1.0 / 10000 ** (np.arange(d // 2, dtype=np.float64) / (d / 2.0))
        out = np.einsum("m,d->md", pos.reshape(-1), om)
        return np.concatenate([np.sin(out), np.cos(out)], axis=1)
    return torch.from_numpy(np.concatenate([one(dim // 2, X), one(dim // 2, Y)], axis=1)).float()


def sd3_oracle(sd, cfg, latents, enc, t, pooled, qk_norm):
    D, H, Dh, L = cfg.inner_dim, cfg.num_attention_heads, cfg.attention_head_dim, cfg.num_layers
    lin = lambda n, x: F.linear(x, sd[n + ".weight"], sd.get(n + ".bias"))
    mlp2 = lambda n, x: lin(n + ".linear_2", F.silu(lin(n + ".linear_1", x)))
    ln = lambda x: F.layer_norm(x, (D,), eps=1e-6)
    rms = lambda x, n: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * sd[n] if qk_norm else x
    B, _, h2, w2 = latents.shape
    x = F.conv2d(latents, sd["pos_embed.proj.weight"], sd["pos_embed.proj.bias"], stride=2).flatten(2).transpose(1, 2)
    h, w, M = h2 // 2, w2 // 2, cfg.pos_embed_max_size
    top, left = (M - h) // 2, (M - w) // 2
    x = x + sd["pos_embed.pos_embed"].view(M, M, D)[top:top + h, left:left + w].reshape(1, h * w, D)
    c = lin("context_embedder", enc)
    st = F.silu(mlp2("time_text_embed.timestep_embedder", _sinus(t)) + mlp2("time_text_embed.text_embedder", pooled))
    heads = lambda y: y.view(B, -1, H, Dh)
    S = x.shape[1]
    for i in range(L):
        p = f"transformer_blocks.{i}."
        pre_only = i == L - 1
        mx = lin(p + "norm1.linear", st).chunk(6, -1)
        xn = ln(x) * (1 + mx[1][:, None]) + mx[0][:, None]
        if pre_only:
            sc, sh = lin(p + "norm1_context.linear", st).chunk(2, -1)
            cn = ln(c) * (1 + sc[:, None]) + sh[:, None]
        else:
            mc = lin(p + "norm1_context.linear", st).chunk(6, -1)
            cn = ln(c) * (1 + mc[1][:, None]) + mc[0][:, None]
        q = torch.cat([rms(heads(lin(p + "attn.to_q", xn)), p + "attn.norm_q.weight"),
                       rms(heads(lin(p + "attn.add_q_proj", cn)), p + "attn.norm_added_q.weight")], 1)
        k = torch.cat([rms(heads(lin(p + "attn.to_k", xn)), p + "attn.norm_k.weight"),
                       rms(heads(lin(p + "attn.add_k_proj", cn)), p + "attn.norm_added_k.weight")], 1)
        v = torch.cat([heads(lin(p + "attn.to_v", xn)), heads(lin(p + "attn.add_v_proj", cn))], 1)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2).reshape(B, -1, D)
        ff = lambda n, y: lin(n + ".net.2", F.gelu(lin(n + ".net.0.proj", y), approximate="tanh"))
        x = x + mx[2][:, None] * lin(p + "attn.to_out.0", o[:, :S])
        x = x + mx[5][:, None] * ff(p + "ff", ln(x) * (1 + mx[4][:, None]) + mx[3][:, None])
        if not pre_only:
            c = c + mc[2][:, None] * lin(p + "attn.to_add_out", o[:, S:])
            c = c + mc[5][:, None] * ff(p + "ff_context", ln(c) * (1 + mc[4][:, None]) + mc[3][:, None])
    scale, shift = lin("norm_out.linear", st).chunk(2, -1)
    out = lin("proj_out", ln(x) * (1 + scale[:, None]) + shift[:, None])              # [B, S, 2*2*C]
    C = out.shape[-1] // 4
    return out.view(B, h, w, 2, 2, C).permute(0, 5, 1, 3, 2, 4).reshape(B, C, h2, w2)  # nhwpqc -> nchpwq


def _run(qk_norm):
    torch.manual_seed(0)
    cfg = SD3TransformerConfig(num_layers=2, attention_head_dim=16, num_attention_heads=4, joint_attention_dim=40,
                               pooled_projection_dim=24, in_channels=16, out_channels=4, pos_embed_max_size=12,
                               qk_norm="rms_norm" if qk_norm else None)
    m = SD3Transformer2DModel(cfg, torch.float32, "cpu", sample_size=16)
    assert torch.allclose(m.pos_table, _pos_table(cfg.inner_dim, 12, 8), atol=1e-6)
    params = dict(m.named_parameters())
    D = cfg.inner_dim
    sd = {}
    for name, (pn, sl) in m.checkpoint_name_map().items():
        base = name.split("#")[0]
        shape = list(params[pn].shape)
        if sl is not None:
            shape[0] = sl[1] - sl[0]
        if base.endswith("norm1_context.linear.weight") and "#" in name:
            shape = [2 * D, D]
        elif base.endswith("norm1_context.linear.bias") and "#" in name:
            shape = [2 * D]
        if base not in sd:
            sd[base] = torch.randn(shape) * 0.08 + (1.0 if ".attn.norm_" in base else 0.0)
    sd["pos_embed.proj.weight"] = sd["pos_embed.proj.weight"].view(D, 4, 2, 2)
    sd["pos_embed.pos_embed"] = m.pos_table.clone()[None]
    assert m.load_weights(sd.items()) == set(sd)
    B, h2, w2, St = 2, 8, 6, 5
    lat, enc = torch.randn(B, 4, h2, w2), torch.randn(B, St, 40)
    t, pooled = torch.tensor([0.7, 0.3]), torch.randn(B, 24)
    with torch.no_grad():
        out = m(pack_latents(lat), enc, t, (1, h2 // 2, w2 // 2), pooled_projections=pooled)
        ref = sd3_oracle(sd, cfg, lat, enc, t, pooled, qk_norm)
    ref_packed = pack_latents(ref)
    assert out.shape == ref_packed.shape
    assert (out - ref_packed).abs().max().item() < 2e-4 * max(1.0, ref.abs().max().item())


def test_sd3_forward_from_diffusers_named_tensors():
    _run(qk_norm=False)


def test_sd35_forward_with_qk_rms_norm():
    _run(qk_norm=True)
