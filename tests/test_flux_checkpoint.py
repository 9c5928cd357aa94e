"""FLUX transformer against a straight-line PyTorch restatement of the published architecture that
works directly on a dict of diffusers-named tensors (``x_embedder``, ``transformer_blocks.N.attn.to_q``,
``single_transformer_blocks.N.proj_mlp`` ...).  Checks the name map (q/k/v + MLP stacking, stacked
modulation layers) and the fused forward in one go."""
import math

import torch
import torch.nn.functional as F

from vllm_omni_b200.diffusion.models.flux.transformer import FluxTransformer2DModel, FluxTransformerConfig


def _sinus(t):
    half = 128
    e = (t.float()[:, None] * 1000.0) * torch.exp(-math.log(10000.0) * torch.arange(half).float() / half)[None]
    return torch.cat([e.cos(), e.sin()], -1)


def _rope_tables(ids, axes, theta=10000.0):
    cs, sn = [], []
    for a, d in enumerate(axes):
        inv = 1.0 / (theta ** (torch.arange(0, d, 2).float() / d))
        ang = ids[:, a].float()[:, None] * inv[None]
        cs.append(ang.cos().repeat_interleave(2, -1))
        sn.append(ang.sin().repeat_interleave(2, -1))
    return torch.cat(cs, -1), torch.cat(sn, -1)


def _rope(x, cos, sin):           # x [B, S, H, D]; pairs (0,1), (2,3), ...
    xr = torch.stack([-x[..., 1::2], x[..., 0::2]], -1).flatten(-2)
    return x * cos[None, :, None] + xr * sin[None, :, None]


def flux_oracle(sd, cfg, hidden, enc, t, pooled, guidance, h, w, ids=None, temb=None):
    """``ids``: [S_txt + h*w, 3] position ids, text rows first (FLUX: zeros for text, (0, y, x) for
    patches).  ``temb``: conditioning vector when it is not FLUX's timestep + guidance + pooled sum."""
    D, H, Dh = cfg.inner_dim, cfg.num_attention_heads, cfg.attention_head_dim
    lin = lambda n, x: F.linear(x, sd[n + ".weight"], sd.get(n + ".bias"))
    mlp2 = lambda n, x: lin(n + ".linear_2", F.silu(lin(n + ".linear_1", x)))
    ln = lambda x: F.layer_norm(x, (D,), eps=1e-6)
    rms = lambda x, n: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * sd[n]
    if temb is None:
        temb = mlp2("time_text_embed.timestep_embedder", _sinus(t)) + mlp2("time_text_embed.guidance_embedder", _sinus(guidance)) \
            + mlp2("time_text_embed.text_embedder", pooled)
    st = F.silu(temb)
    x, c = lin("x_embedder", hidden), lin("context_embedder", enc)
    B, Si, St = x.shape[0], x.shape[1], c.shape[1]
    if ids is None:
        ys, xs = torch.arange(h).repeat_interleave(w), torch.arange(w).repeat(h)
        ids = torch.cat([torch.zeros(St, 3), torch.stack([torch.zeros(h * w), ys.float(), xs.float()], -1)])
    cos, sin = _rope_tables(ids, cfg.axes_dims_rope)
    heads = lambda y: y.view(B, -1, H, Dh)

    def attend(q, k, v):
        q, k = _rope(q, cos, sin), _rope(k, cos, sin)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
        return o.transpose(1, 2).reshape(B, -1, D)

    for i in range(cfg.num_layers):
        p = f"transformer_blocks.{i}."
        mx = lin(p + "norm1.linear", st).chunk(6, -1)
        mc = lin(p + "norm1_context.linear", st).chunk(6, -1)
        xn = ln(x) * (1 + mx[1][:, None]) + mx[0][:, None]
        cn = ln(c) * (1 + mc[1][:, None]) + mc[0][:, None]
        q = torch.cat([rms(heads(lin(p + "attn.add_q_proj", cn)), p + "attn.norm_added_q.weight"),
                       rms(heads(lin(p + "attn.to_q", xn)), p + "attn.norm_q.weight")], 1)
        k = torch.cat([rms(heads(lin(p + "attn.add_k_proj", cn)), p + "attn.norm_added_k.weight"),
                       rms(heads(lin(p + "attn.to_k", xn)), p + "attn.norm_k.weight")], 1)
        v = torch.cat([heads(lin(p + "attn.add_v_proj", cn)), heads(lin(p + "attn.to_v", xn))], 1)
        o = attend(q, k, v)
        x = x + mx[2][:, None] * lin(p + "attn.to_out.0", o[:, St:])
        c = c + mc[2][:, None] * lin(p + "attn.to_add_out", o[:, :St])
        ff = lambda n, y: lin(n + ".net.2", F.gelu(lin(n + ".net.0.proj", y), approximate="tanh"))
        x = x + mx[5][:, None] * ff(p + "ff", ln(x) * (1 + mx[4][:, None]) + mx[3][:, None])
        c = c + mc[5][:, None] * ff(p + "ff_context", ln(c) * (1 + mc[4][:, None]) + mc[3][:, None])
    y = torch.cat([c, x], 1)
    for i in range(cfg.num_single_layers):
        p = f"single_transformer_blocks.{i}."
        sh, sc, g = lin(p + "norm.linear", st).chunk(3, -1)
        yn = ln(y) * (1 + sc[:, None]) + sh[:, None]
        q = rms(heads(lin(p + "attn.to_q", yn)), p + "attn.norm_q.weight")
        k = rms(heads(lin(p + "attn.to_k", yn)), p + "attn.norm_k.weight")
        o = attend(q, k, heads(lin(p + "attn.to_v", yn)))
        m = F.gelu(lin(p + "proj_mlp", yn), approximate="tanh")
        y = y + g[:, None] * lin(p + "proj_out", torch.cat([o, m], -1))
    x = y[:, St:]
    scale, shift = lin("norm_out.linear", st).chunk(2, -1)
    return lin("proj_out", ln(x) * (1 + scale[:, None]) + shift[:, None])


def test_flux_forward_from_diffusers_named_tensors():
    torch.manual_seed(0)
    cfg = FluxTransformerConfig(num_layers=2, num_single_layers=2, attention_head_dim=32, num_attention_heads=2,
                                joint_attention_dim=48, pooled_projection_dim=24, axes_dims_rope=(8, 12, 12), in_channels=16,
                                out_channels=4)
    m = FluxTransformer2DModel(cfg, torch.float32, "cpu")
    params = dict(m.named_parameters())
    sd = {}
    for name, (pn, sl) in m.checkpoint_name_map().items():
        shape = list(params[pn].shape)
        if sl is not None:
            shape[0] = sl[1] - sl[0]
        sd[name] = torch.randn(shape) * 0.08 + (1.0 if ("attn.norm_" in name) else 0.0)
    assert m.load_weights(sd.items()) == set(sd)
    B, h, w, St = 2, 4, 6, 5
    hidden, enc = torch.randn(B, h * w, 16), torch.randn(B, St, 48)
    t, pooled, g = torch.tensor([0.7, 0.3]), torch.randn(B, 24), torch.tensor([3.5, 2.0])
    with torch.no_grad():
        out = m(hidden, enc, t, (1, h, w), pooled_projections=pooled, guidance=g)
        ref = flux_oracle(sd, cfg, hidden, enc, t, pooled, g, h, w)
    assert out.shape == ref.shape == (B, h * w, 16)
    assert (out - ref).abs().max().item() < 2e-4 * max(1.0, ref.abs().max().item())


def test_longcat_forward_from_checkpoint_named_tensors():
    """LongCat-Image: FLUX blocks conditioned on the timestep alone, position ids with a modality axis
    (text (0, i, i), image (1, y + 512, x + 512))."""
    from vllm_omni_b200.diffusion.models.longcat_image.transformer import LongCatImageTransformer2DModel, LongCatTransformerConfig
    torch.manual_seed(0)
    cfg = LongCatTransformerConfig(num_layers=1, num_single_layers=2, attention_head_dim=32, num_attention_heads=2,
                                   joint_attention_dim=48, axes_dims_rope=(8, 12, 12), in_channels=16, out_channels=4)
    m = LongCatImageTransformer2DModel(cfg, torch.float32, "cpu")
    params = dict(m.named_parameters())
    sd = {}
    for name, (pn, sl) in m.checkpoint_name_map().items():
        shape = list(params[pn].shape)
        if sl is not None:
            shape[0] = sl[1] - sl[0]
        sd[name] = torch.randn(shape) * 0.08 + (1.0 if ("attn.norm_" in name) else 0.0)
    assert m.load_weights(sd.items()) == set(sd) and not any(k.startswith("time_text_embed") for k in sd)
    B, h, w, St = 2, 4, 6, 5
    hidden, enc, t = torch.randn(B, h * w, 16), torch.randn(B, St, 48), torch.tensor([0.7, 0.3])
    ys, xs = torch.arange(h).repeat_interleave(w) + 512, torch.arange(w).repeat(h) + 512
    ti = torch.arange(St).float()
    ids = torch.cat([torch.stack([torch.zeros(St), ti, ti], -1), torch.stack([torch.ones(h * w), ys.float(), xs.float()], -1)])
    lin = lambda n, x: F.linear(x, sd[n + ".weight"], sd[n + ".bias"])
    temb = lin("time_embed.timestep_embedder.linear_2", F.silu(lin("time_embed.timestep_embedder.linear_1", _sinus(t))))
    with torch.no_grad():
        out = m(hidden, enc, t, (1, h, w))
        ref = flux_oracle(sd, cfg, hidden, enc, t, None, None, h, w, ids=ids, temb=temb)
    assert (out - ref).abs().max().item() < 2e-4 * max(1.0, ref.abs().max().item())


def ovis_oracle(sd, cfg, hidden, enc, t, h, w):
    D, H, Dh = cfg.inner_dim, cfg.num_attention_heads, cfg.attention_head_dim
    lin = lambda n, x: F.linear(x, sd[n + ".weight"], sd.get(n + ".bias"))
    ln = lambda x: F.layer_norm(x, (D,), eps=1e-6)
    rms = lambda x, w_: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w_
    st = F.silu(lin("timestep_embedder.linear_2", F.silu(lin("timestep_embedder.linear_1", _sinus(t)))))
    x = lin("x_embedder", hidden)
    c = lin("context_embedder", rms(enc, sd["context_embedder_norm.weight"]))
    B, St = x.shape[0], c.shape[1]
    ys, xs = torch.arange(h).repeat_interleave(w).float(), torch.arange(w).repeat(h).float()
    ti = torch.arange(St).float()
    ids = torch.cat([torch.stack([torch.zeros(St), ti, ti], -1), torch.stack([torch.zeros(h * w), ys, xs], -1)])
    cos, sin = _rope_tables(ids, cfg.axes_dims_rope)
    heads = lambda y: y.view(B, -1, H, Dh)

    def attend(q, k, v):
        o = F.scaled_dot_product_attention(_rope(q, cos, sin).transpose(1, 2), _rope(k, cos, sin).transpose(1, 2), v.transpose(1, 2))
        return o.transpose(1, 2).reshape(B, -1, D)

    def swiglu_ff(n, y):
        val, gate = lin(n + ".net.0.proj", y).chunk(2, -1)
        return lin(n + ".net.2", val * F.silu(gate))
    for i in range(cfg.num_layers):
        p = f"transformer_blocks.{i}."
        mx, mc = lin(p + "norm1.linear", st).chunk(6, -1), lin(p + "norm1_context.linear", st).chunk(6, -1)
        xn, cn = ln(x) * (1 + mx[1][:, None]) + mx[0][:, None], ln(c) * (1 + mc[1][:, None]) + mc[0][:, None]
        q = torch.cat([rms(heads(lin(p + "attn.add_q_proj", cn)), sd[p + "attn.norm_added_q.weight"]),
                       rms(heads(lin(p + "attn.to_q", xn)), sd[p + "attn.norm_q.weight"])], 1)
        k = torch.cat([rms(heads(lin(p + "attn.add_k_proj", cn)), sd[p + "attn.norm_added_k.weight"]),
                       rms(heads(lin(p + "attn.to_k", xn)), sd[p + "attn.norm_k.weight"])], 1)
        v = torch.cat([heads(lin(p + "attn.add_v_proj", cn)), heads(lin(p + "attn.to_v", xn))], 1)
        o = attend(q, k, v)
        x = x + mx[2][:, None] * lin(p + "attn.to_out.0", o[:, St:])
        c = c + mc[2][:, None] * lin(p + "attn.to_add_out", o[:, :St])
        x = x + mx[5][:, None] * swiglu_ff(p + "ff", ln(x) * (1 + mx[4][:, None]) + mx[3][:, None])
        c = c + mc[5][:, None] * swiglu_ff(p + "ff_context", ln(c) * (1 + mc[4][:, None]) + mc[3][:, None])
    y = torch.cat([c, x], 1)
    for i in range(cfg.num_single_layers):
        p = f"single_transformer_blocks.{i}."
        sh, sc, g = lin(p + "norm.linear", st).chunk(3, -1)
        yn = ln(y) * (1 + sc[:, None]) + sh[:, None]
        mlp, gate = lin(p + "proj_mlp", yn).chunk(2, -1)
        q = rms(heads(lin(p + "attn.to_q", yn)), sd[p + "attn.norm_q.weight"])
        k = rms(heads(lin(p + "attn.to_k", yn)), sd[p + "attn.norm_k.weight"])
        o = attend(q, k, heads(lin(p + "attn.to_v", yn)))
        y = y + g[:, None] * lin(p + "proj_out", torch.cat([o, F.silu(gate) * mlp], -1))
    scale, shift = lin("norm_out.linear", st).chunk(2, -1)
    return lin("proj_out", ln(y[:, St:]) * (1 + scale[:, None]) + shift[:, None])


def test_ovis_forward_from_checkpoint_named_tensors():
    from vllm_omni_b200.diffusion.models.ovis_image.transformer import OvisImageTransformer2DModel, OvisTransformerConfig
    torch.manual_seed(0)
    cfg = OvisTransformerConfig(num_layers=1, num_single_layers=2, attention_head_dim=32, num_attention_heads=2,
                                joint_attention_dim=48, axes_dims_rope=(8, 12, 12), in_channels=16, out_channels=4)
    m = OvisImageTransformer2DModel(cfg, torch.float32, "cpu")
    params = dict(m.named_parameters())
    sd, covered = {}, {}
    for name, (pn, sl) in m.checkpoint_name_map().items():
        shape = list(params[pn].shape)
        if sl is not None:
            shape[0] = sl[1] - sl[0]
        covered[pn] = covered.get(pn, 0) + shape[0]
        sd[name] = torch.randn(shape) * 0.08 + (1.0 if ("attn.norm_" in name or "embedder_norm" in name) else 0.0)
    assert all(covered.get(pn) == p.shape[0] for pn, p in params.items())
    assert m.load_weights(sd.items()) == set(sd)
    B, h, w, St = 2, 4, 6, 5
    hidden, enc, t = torch.randn(B, h * w, 16), torch.randn(B, St, 48), torch.tensor([0.7, 0.3])
    with torch.no_grad():
        out = m(hidden, enc, t, (1, h, w))
        ref = ovis_oracle(sd, cfg, hidden, enc, t, h, w)
    assert (out - ref).abs().max().item() < 2e-4 * max(1.0, ref.abs().max().item())
