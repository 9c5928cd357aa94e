"""GLM-Image DiT against a straight-line PyTorch restatement on diffusers-named tensors: prior-token
embedding with CFG drop, twelve-way modulation, ONE attention with shared weights over [text | image]
(affine-free LayerNorm on q / k heads, 2-D rotary embedding on the image rows only), ONE shared
feed-forward, size conditioning; plus the key / value cache of the editing mode."""
import math

import torch
import torch.nn.functional as F

from vllm_omni_b200.diffusion.models.glm_image.transformer import (GlmImageKVCache, GlmImageTransformer2DModel,
                                                                    GlmImageTransformerConfig)


def _sin(x, dim):
    half = dim // 2
    a = x.float()[:, None] * torch.exp(-math.log(10000.0) * torch.arange(half).float() / half)[None]
    return torch.cat([a.cos(), a.sin()], -1)


def oracle(sd, c, lat, enc, prior, drop, t, target, crop, cached=None, store=None):
    D, H, Dh, p = c.inner_dim, c.num_attention_heads, c.attention_head_dim, c.patch_size
    lin = lambda n, x: F.linear(x, sd[n + ".weight"], sd[n + ".bias"])
    B, C, Hh, Ww = lat.shape
    x = lat.reshape(B, C, Hh // p, p, Ww // p, p).permute(0, 2, 4, 1, 3, 5).flatten(3, 5).flatten(1, 2)
    x = lin("image_projector.proj", x)
    txt = lin("glyph_projector.net.2", F.gelu(lin("glyph_projector.net.0.proj", enc)))
    pe = sd["prior_token_embedding.weight"][prior].clone()
    pe[drop] *= 0.0
    x = x + lin("prior_projector.net.2", F.silu(lin("prior_projector.net.0.proj", pe)))
    mlp = lambda n, y: lin(n + ".linear_2", F.silu(lin(n + ".linear_1", y)))
    cond = torch.cat([_sin(crop.flatten(), c.condition_dim).view(B, -1), _sin(target.flatten(), c.condition_dim).view(B, -1)], 1)
    temb = mlp("time_condition_embed.timestep_embedder", _sin(t, c.time_embed_dim)) + mlp("time_condition_embed.condition_embedder", cond)
    h, w = Hh // p, Ww // p
    d = Dh // 2
    inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2).float()[: d // 2] / d))
    fr = torch.cat([torch.outer(torch.arange(h).float(), inv)[:, None].expand(h, w, -1),
                    torch.outer(torch.arange(w).float(), inv)[None].expand(h, w, -1)], -1)
    fr = torch.cat([fr, fr], -1).reshape(h * w, Dh)
    cos, sin = fr.cos()[None, :, None], fr.sin()[None, :, None]

    def rope(y):                                   # halves: (first, second) = (real, imaginary)
        re, im = y.reshape(*y.shape[:-1], 2, -1).unbind(-2)
        return y * cos + torch.cat([-im, re], -1) * sin
    ln = lambda y: F.layer_norm(y, (D,), eps=1e-5)
    St = txt.shape[1]
    for i in range(c.num_layers):
        b = f"transformer_blocks.{i}."
        m = lin(b + "norm1.linear", temb).chunk(12, 1)
        sh, csh, sc, csc, g, cg, sh2, csh2, sc2, csc2, g2, cg2 = (v[:, None] for v in m)
        u = torch.cat([ln(txt) * (1 + csc) + csh, ln(x) * (1 + sc) + sh], 1)
        q = F.layer_norm(lin(b + "attn1.to_q", u).unflatten(-1, (H, Dh)), (Dh,), eps=1e-5)
        k = F.layer_norm(lin(b + "attn1.to_k", u).unflatten(-1, (H, Dh)), (Dh,), eps=1e-5)
        v = lin(b + "attn1.to_v", u).unflatten(-1, (H, Dh))
        q = torch.cat([q[:, :St], rope(q[:, St:])], 1)
        k = torch.cat([k[:, :St], rope(k[:, St:])], 1)
        if store is not None:
            store.append((k.clone(), v.clone()))
        if cached is not None:
            k, v = torch.cat([cached[i][0], k], 1), torch.cat([cached[i][1], v], 1)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2).flatten(2)
        o = lin(b + "attn1.to_out.0", o)
        txt, x = txt + o[:, :St] * cg, x + o[:, St:] * g
        ff = lambda y: lin(b + "ff.net.2", F.gelu(lin(b + "ff.net.0.proj", y), approximate="tanh"))
        x = x + ff(ln(x) * (1 + sc2) + sh2) * g2
        txt = txt + ff(ln(txt) * (1 + csc2) + csh2) * cg2
    scale, shift = lin("norm_out.linear", temb).chunk(2, 1)
    y = lin("proj_out", ln(x) * (1 + scale)[:, None] + shift[:, None])
    return y.reshape(B, h, w, -1, p, p).permute(0, 3, 1, 4, 2, 5).flatten(4, 5).flatten(2, 3)


def _model():
    torch.manual_seed(0)
    c = GlmImageTransformerConfig(num_layers=2, attention_head_dim=16, num_attention_heads=2, time_embed_dim=32, condition_dim=8,
                                  prior_vq_quantizer_codebook_size=20, text_embed_dim=24, in_channels=4, out_channels=4)
    m = GlmImageTransformer2DModel(c, torch.float32, "cpu")
    D = c.inner_dim
    sd = {}
    for n, p in m.named_parameters():
        if ".attn1.to_qkv." in n:
            for i, s in enumerate(("to_q", "to_k", "to_v")):
                sd[n.replace("to_qkv", s)] = torch.randn(D, *p.shape[1:]) * 0.1
        else:
            sd[n] = torch.randn(p.shape) * 0.1
    assert m.load_weights(sd.items()) == set(sd)
    return c, m, sd


def test_glm_image_forward_from_diffusers_named_tensors():
    c, m, sd = _model()
    B, Hh, Ww, St = 2, 8, 12, 5
    lat, enc = torch.randn(B, 4, Hh, Ww), torch.randn(B, St, 24)
    prior = torch.randint(0, 20, (B, 24))
    drop = torch.zeros(B, 24, dtype=torch.bool)
    drop[1] = True                                           # the unconditional row drops its prior tokens
    t, target, crop = torch.tensor([700.0, 250.0]), torch.tensor([[64.0, 96.0]] * 2), torch.zeros(B, 2)
    with torch.no_grad():
        out = m(lat, enc, prior, drop, t, target, crop)
        ref = oracle(sd, c, lat, enc, prior, drop, t, target, crop)
    assert out.shape == ref.shape == (B, 4, Hh, Ww)
    assert (out - ref).abs().max().item() < 2e-4 * max(1.0, ref.abs().max().item())


def test_glm_image_condition_kv_cache_write_then_read():
    c, m, sd = _model()
    Hh, Ww, St = 8, 8, 4
    cond_lat, lat, enc = torch.randn(1, 4, Hh, Ww), torch.randn(1, 4, Hh, Ww), torch.randn(1, St, 24)
    prior, keep = torch.randint(0, 20, (1, 16)), torch.zeros(1, 16, dtype=torch.bool)
    target, crop = torch.tensor([[64.0, 64.0]]), torch.zeros(1, 2)
    cache = GlmImageKVCache(c.num_layers)
    with torch.no_grad():
        cache.mode = "write"
        m(cond_lat, enc, prior, keep, torch.zeros(1), target, crop, kv_cache=cache)
        cache.mode = "read"
        out = m(lat, enc, prior, keep, torch.tensor([500.0]), target, crop, kv_cache=cache)
        stored = []
        oracle(sd, c, cond_lat, enc, prior, keep, torch.zeros(1), target, crop, store=stored)
        ref = oracle(sd, c, lat, enc, prior, keep, torch.tensor([500.0]), target, crop, cached=stored)
        plain = m(lat, enc, prior, keep, torch.tensor([500.0]), target, crop)
    assert (out - ref).abs().max().item() < 2e-4 * max(1.0, ref.abs().max().item())
    assert (out - plain).abs().max().item() > 1e-4                      # the condition image does change the prediction
    cache.clear()
    assert cache.layers[0].k is None and cache.mode is None
