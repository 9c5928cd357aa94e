"""Z-Image transformer against a straight-line PyTorch restatement of the published architecture on
a dict of checkpoint-named tensors (``all_x_embedder.2-1``, ``noise_refiner.N.attention.to_q``,
``layers.N.feed_forward.w1`` ...): pad tokens, refiners, unified sequence, 3-axis rotary positions
that depend on the caption length, tanh gates, final layer."""
import math

import torch
import torch.nn.functional as F

from vllm_omni_b200.diffusion.models.z_image.transformer import ZImageTransformer2DModel, ZImageTransformerConfig


def oracle(sd, c, image, cap_feat, t):
    """One sample: image [C, F, H, W], cap_feat [L, cap_dim], t scalar.  Returns [C, F, H, W]."""
    D, H, Dh = c.dim, c.n_heads, c.head_dim
    lin = lambda n, x: F.linear(x, sd[n + ".weight"], sd.get(n + ".bias"))
    rms = lambda x, w, eps=c.norm_eps: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w
    half = 128
    fr = torch.exp(-math.log(10000.0) * torch.arange(half).float() / half)
    a = (t * c.t_scale) * fr
    temb = lin("t_embedder.mlp.2", F.silu(lin("t_embedder.mlp.0", torch.cat([a.cos(), a.sin()])[None])))[0]

    def rope_tables(ids):
        cs, sn = [], []
        for ax, d in enumerate(c.axes_dims):
            inv = 1.0 / (c.rope_theta ** (torch.arange(0, d, 2).double() / d))
            ang = torch.outer(ids[:, ax].double(), inv).float()
            cs.append(ang.cos()), sn.append(ang.sin())
        return torch.cat(cs, -1).repeat_interleave(2, -1), torch.cat(sn, -1).repeat_interleave(2, -1)

    def rope(x, cos, sin):          # [S, H, Dh], interleaved pairs
        xr = torch.stack([-x[..., 1::2], x[..., 0::2]], -1).flatten(-2)
        return x * cos[:, None] + xr * sin[:, None]

    def block(p, x, cos, sin, mod):
        if mod:
            s1, g1, s2, g2 = lin(p + "adaLN_modulation.0", temb[None])[0].chunk(4)
            s1, s2, g1, g2 = 1 + s1, 1 + s2, g1.tanh(), g2.tanh()
        else:
            s1 = s2 = g1 = g2 = 1.0
        h = rms(x, sd[p + "attention_norm1.weight"]) * s1
        q = rms(lin(p + "attention.to_q", h).view(-1, H, Dh), sd[p + "attention.norm_q.weight"])
        k = rms(lin(p + "attention.to_k", h).view(-1, H, Dh), sd[p + "attention.norm_k.weight"])
        v = lin(p + "attention.to_v", h).view(-1, H, Dh)
        o = F.scaled_dot_product_attention(rope(q, cos, sin).transpose(0, 1), rope(k, cos, sin).transpose(0, 1), v.transpose(0, 1))
        x = x + g1 * rms(lin(p + "attention.to_out.0", o.transpose(0, 1).reshape(-1, D)), sd[p + "attention_norm2.weight"])
        h = rms(x, sd[p + "ffn_norm1.weight"]) * s2
        f = lin(p + "feed_forward.w2", F.silu(lin(p + "feed_forward.w1", h)) * lin(p + "feed_forward.w3", h))
        return x + g2 * rms(f, sd[p + "ffn_norm2.weight"])

    C, Fr, Hh, Ww = image.shape
    ps = c.patch_size
    L = cap_feat.shape[0]
    Lp = L + (-L) % 32
    cap_ids = torch.stack([torch.arange(1, Lp + 1), torch.zeros(Lp), torch.zeros(Lp)], -1).long()
    x = image.view(C, Fr, 1, Hh // ps, ps, Ww // ps, ps).permute(1, 3, 5, 2, 4, 6, 0).reshape(-1, ps * ps * C)
    S = x.shape[0]
    Sp = S + (-S) % 32
    g = torch.stack(torch.meshgrid(torch.arange(Fr), torch.arange(Hh // ps), torch.arange(Ww // ps), indexing="ij"), -1).reshape(-1, 3)
    x_ids = torch.cat([g + torch.tensor([Lp + 1, 0, 0]), torch.zeros(Sp - S, 3).long()])
    x = torch.cat([lin("all_x_embedder.2-1", x), sd["x_pad_token"].expand(Sp - S, -1)])
    xc, xs = rope_tables(x_ids)
    for i in range(c.n_refiner_layers):
        x = block(f"noise_refiner.{i}.", x, xc, xs, True)
    cap = lin("cap_embedder.1", rms(cap_feat, sd["cap_embedder.0.weight"]))
    cap = torch.cat([cap, sd["cap_pad_token"].expand(Lp - L, -1)])
    cc, cs_ = rope_tables(cap_ids)
    for i in range(c.n_refiner_layers):
        cap = block(f"context_refiner.{i}.", cap, cc, cs_, False)
    u, uc, us = torch.cat([x, cap]), torch.cat([xc, cc]), torch.cat([xs, cs_])
    for i in range(c.n_layers):
        u = block(f"layers.{i}.", u, uc, us, True)
    scale = 1 + lin("all_final_layer.2-1.adaLN_modulation.1", F.silu(temb)[None])[0]
    out = lin("all_final_layer.2-1.linear", F.layer_norm(u, (D,), eps=1e-6) * scale)[:S]
    return out.view(Fr, Hh // ps, Ww // ps, 1, ps, ps, C).permute(6, 0, 3, 1, 4, 2, 5).reshape(C, Fr, Hh, Ww)


def test_z_image_forward_from_checkpoint_named_tensors():
    torch.manual_seed(0)
    c = ZImageTransformerConfig(dim=64, n_layers=2, n_refiner_layers=1, n_heads=4, n_kv_heads=4, in_channels=4,
                                cap_feat_dim=24, axes_dims=(4, 6, 6), axes_lens=(256, 32, 32))
    m = ZImageTransformer2DModel(c, torch.float32, "cpu")
    params = dict(m.named_parameters())
    nmap = m.checkpoint_name_map()
    covered = {}
    sd = {}
    for name, (pn, sl) in nmap.items():
        shape = list(params[pn].shape)
        if sl is not None:
            shape[0] = sl[1] - sl[0]
        covered[pn] = covered.get(pn, 0) + shape[0]
        sd[name] = torch.randn(shape) * 0.1 + (1.0 if "norm" in name or name == "cap_embedder.0.weight" else 0.0)
    assert all(covered.get(pn) == p.shape[0] for pn, p in params.items()), "every parameter has a checkpoint source"
    assert m.load_weights(sd.items()) == set(sd)
    B, Hh, Ww = 2, 12, 10                       # 6 x 5 = 30 patches -> 2 pad tokens
    lat = torch.randn(B, 4, Hh, Ww)
    caps = [torch.randn(40, 24), torch.randn(5, 24)]          # 64 and 32 rows with pad tokens
    enc = torch.zeros(B, 40, 24)
    enc[0], enc[1, :5] = caps[0], caps[1]
    t = torch.tensor([0.3, 0.8])
    with torch.no_grad():
        out = m.unpatchify(m(m.patchify(lat), enc, t, (1, Hh // 2, Ww // 2), txt_seq_lens=[40, 5]), 1, Hh, Ww)
        for b in range(B):
            ref = oracle(sd, c, lat[b][:, None], caps[b], t[b])
            assert (out[b] - ref).abs().max().item() < 2e-4 * max(1.0, ref.abs().max().item()), b
    # patch layout round trip
    assert torch.equal(m.unpatchify(m.patchify(lat), 1, Hh, Ww)[:, :, 0], lat)
