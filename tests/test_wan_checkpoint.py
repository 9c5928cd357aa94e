"""Wan video DiT against a straight-line PyTorch restatement of the published architecture on a dict
of diffusers-named tensors: Conv3d patch embedding, per-block ``scale_shift_table`` + timestep
projection, self attention with full-width q/k RMSNorm and 3-axis complex rotary embedding, cross
attention to the text states, GELU FFN, modulated output layer, patch-major un-patchify."""
import math

import torch
import torch.nn.functional as F

from vllm_omni_b200.diffusion.models.wan.transformer import WanTransformer3DModel, WanTransformerConfig


def wan_oracle(sd, cfg, x, t, enc):
    D, H, Dh = cfg.inner_dim, cfg.num_attention_heads, cfg.attention_head_dim
    lin = lambda n, y: F.linear(y, sd[n + ".weight"], sd.get(n + ".bias"))
    ln = lambda y: F.layer_norm(y.float(), (D,), eps=cfg.eps)
    rms = lambda y, n: y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + cfg.eps) * sd[n]
    B, C, T, Hh, Ww = x.shape
    pt, ph, pw = cfg.patch_size
    f, h, w = T // pt, Hh // ph, Ww // pw
    tok = F.conv3d(x, sd["patch_embedding.weight"], sd["patch_embedding.bias"], stride=cfg.patch_size).flatten(2).transpose(1, 2)
    half = cfg.freq_dim // 2
    a = t.float()[:, None] * torch.exp(-math.log(10000.0) * torch.arange(half).float() / half)[None]
    temb = lin("condition_embedder.time_embedder.linear_2", F.silu(lin("condition_embedder.time_embedder.linear_1",
                                                                         torch.cat([a.cos(), a.sin()], -1))))
    e6 = lin("condition_embedder.time_proj", F.silu(temb)).view(B, 6, D)
    ctx = lin("condition_embedder.text_embedder.linear_2", F.gelu(lin("condition_embedder.text_embedder.linear_1", enc),
                                                                  approximate="tanh"))
    # complex rotary table: frequencies split (t, h, w) = (Dh - 2*(Dh//3) ... ) as in WanRotaryPosEmbed
    dh = dw = 2 * (Dh // 6)
    dt = Dh - dh - dw
    def freqs(n, dim):
        inv = 1.0 / (10000.0 ** (torch.arange(0, dim, 2).double() / dim))
        return torch.polar(torch.ones(n, dim // 2, dtype=torch.float64), torch.outer(torch.arange(n).double(), inv))
    fr = torch.cat([freqs(f, dt)[:, None, None].expand(f, h, w, -1), freqs(h, dh)[None, :, None].expand(f, h, w, -1),
                    freqs(w, dw)[None, None, :].expand(f, h, w, -1)], -1).reshape(1, f * h * w, 1, Dh // 2)
    def rope(y):          # [B, S, H, Dh]
        yc = torch.view_as_complex(y.double().reshape(*y.shape[:-1], -1, 2))
        return torch.view_as_real(yc * fr).flatten(-2).float()
    heads = lambda y: y.view(B, -1, H, Dh)
    sdpa = lambda q, k, v: F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2).reshape(B, -1, D)
    for i in range(cfg.num_layers):
        p = f"blocks.{i}."
        sh1, sc1, g1, sh2, sc2, g2 = (sd[p + "scale_shift_table"].float() + e6.float()).chunk(6, dim=1)
        xn = ln(tok) * (1 + sc1) + sh1
        q, k = rms(lin(p + "attn1.to_q", xn), p + "attn1.norm_q.weight"), rms(lin(p + "attn1.to_k", xn), p + "attn1.norm_k.weight")
        o = sdpa(rope(heads(q)), rope(heads(k)), heads(lin(p + "attn1.to_v", xn)))
        tok = tok + lin(p + "attn1.to_out.0", o) * g1
        xn = ln(tok) * sd[p + "norm2.weight"] + sd[p + "norm2.bias"]
        q = rms(lin(p + "attn2.to_q", xn), p + "attn2.norm_q.weight")
        k = rms(lin(p + "attn2.to_k", ctx), p + "attn2.norm_k.weight")
        tok = tok + lin(p + "attn2.to_out.0", sdpa(heads(q), heads(k), heads(lin(p + "attn2.to_v", ctx))))
        xn = ln(tok) * (1 + sc2) + sh2
        tok = tok + lin(p + "ffn.net.2", F.gelu(lin(p + "ffn.net.0.proj", xn), approximate="tanh")) * g2
    shift, scale = (sd["scale_shift_table"].float() + temb[:, None].float()).chunk(2, dim=1)
    y = lin("proj_out", ln(tok) * (1 + scale) + shift)
    return y.reshape(B, f, h, w, pt, ph, pw, -1).permute(0, 7, 1, 4, 2, 5, 3, 6).reshape(B, -1, T, Hh, Ww)


def test_wan_forward_from_diffusers_named_tensors():
    torch.manual_seed(0)
    cfg = WanTransformerConfig(num_layers=2, num_attention_heads=2, attention_head_dim=24, ffn_dim=64, text_dim=32,
                               in_channels=4, out_channels=4)
    m = WanTransformer3DModel(cfg, torch.float32, "cpu")
    D = cfg.inner_dim
    names = {"patch_embedding.weight": (D, 4, 1, 2, 2), "patch_embedding.bias": (D,), "scale_shift_table": (1, 2, D),
             "proj_out.weight": (16, D), "proj_out.bias": (16,), "condition_embedder.time_proj.weight": (6 * D, D),
             "condition_embedder.time_proj.bias": (6 * D,)}
    for n, (i, o) in (("condition_embedder.text_embedder.linear_1", (32, D)), ("condition_embedder.text_embedder.linear_2", (D, D)),
                      ("condition_embedder.time_embedder.linear_1", (256, D)), ("condition_embedder.time_embedder.linear_2", (D, D))):
        names[n + ".weight"], names[n + ".bias"] = (o, i), (o,)
    for i in range(2):
        p = f"blocks.{i}."
        names[p + "scale_shift_table"] = (1, 6, D)
        for a in ("attn1", "attn2"):
            for q in ("to_q", "to_k", "to_v", "to_out.0"):
                names[p + f"{a}.{q}.weight"], names[p + f"{a}.{q}.bias"] = (D, D), (D,)
            names[p + f"{a}.norm_q.weight"], names[p + f"{a}.norm_k.weight"] = (D,), (D,)
        names[p + "norm2.weight"], names[p + "norm2.bias"] = (D,), (D,)
        names[p + "ffn.net.0.proj.weight"], names[p + "ffn.net.0.proj.bias"] = (64, D), (64,)
        names[p + "ffn.net.2.weight"], names[p + "ffn.net.2.bias"] = (D, 64), (D,)
    sd = {n: torch.randn(s) * 0.1 + (1.0 if "norm" in n and n.endswith("weight") else 0.0) for n, s in names.items()}
    assert m.load_weights(sd.items()) == set(sd)
    x, t, enc = torch.randn(2, 4, 3, 8, 6), torch.tensor([900.0, 250.0]), torch.randn(2, 7, 32)
    with torch.no_grad():
        out = m(x, t, enc)
        ref = wan_oracle(sd, cfg, x, t, enc)
    assert out.shape == ref.shape == x.shape
    assert (out - ref).abs().max().item() < 2e-4 * max(1.0, ref.abs().max().item())
