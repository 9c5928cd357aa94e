"""BAGEL's mixture-of-transformers denoiser against a straight-line restatement of the published
packed algorithm (marker rows around the latent rows, understanding weights on the markers,
``*_moe_gen`` weights on the latents, one shared rotary position, context keys in front) on a dict of
checkpoint-named tensors; the understanding-mode prefill; guidance and schedule helpers; the stage."""
import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from vllm_omni_b200.diffusion.models.bagel.mot import BagelMoT, BagelMoTConfig, latent_position_ids, sincos_2d_table
from vllm_omni_b200.diffusion.models.bagel.pipeline import guided_velocity, shifted_time_grid

CFG = BagelMoTConfig(vocab_size=64, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                     intermediate_size=48, max_latent_size=8, z_channels=4, start_of_image=60, end_of_image=61, bos_token_id=58,
                     eos_token_id=59)


def _checkpoint(c):
    D, H, Hkv, Dh, Fi = c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim, c.intermediate_size
    g = lambda *s: torch.randn(*s) * 0.15
    sd = {"language_model.model.embed_tokens.weight": g(c.vocab_size, D), "language_model.model.norm.weight": 1 + g(D),
          "language_model.model.norm_moe_gen.weight": 1 + g(D), "language_model.lm_head.weight": g(c.vocab_size, D),
          "time_embedder.mlp.0.weight": g(D, 256), "time_embedder.mlp.0.bias": g(D), "time_embedder.mlp.2.weight": g(D, D),
          "time_embedder.mlp.2.bias": g(D), "vae2llm.weight": g(D, c.patch_latent_dim), "vae2llm.bias": g(D),
          "llm2vae.weight": g(c.patch_latent_dim, D), "llm2vae.bias": g(c.patch_latent_dim),
          "latent_pos_embed.pos_embed": sincos_2d_table(D, c.max_latent_size), "connector.fc1.weight": g(4, 4)}
    for i in range(c.num_hidden_layers):
        for sfx in ("", "_moe_gen"):
            p = f"language_model.model.layers.{i}."
            for n, rows in (("q_proj", H * Dh), ("k_proj", Hkv * Dh), ("v_proj", Hkv * Dh)):
                sd[p + f"self_attn.{n}{sfx}.weight"], sd[p + f"self_attn.{n}{sfx}.bias"] = g(rows, D), g(rows)
            sd[p + f"self_attn.o_proj{sfx}.weight"] = g(D, H * Dh)
            sd[p + f"self_attn.q_norm{sfx}.weight"], sd[p + f"self_attn.k_norm{sfx}.weight"] = 1 + g(Dh), 1 + g(Dh)
            sd[p + f"mlp{sfx}.gate_proj.weight"], sd[p + f"mlp{sfx}.up_proj.weight"] = g(Fi, D), g(Fi, D)
            sd[p + f"mlp{sfx}.down_proj.weight"] = g(D, Fi)
            sd[p + f"input_layernorm{sfx}.weight"], sd[p + f"post_attention_layernorm{sfx}.weight"] = 1 + g(D), 1 + g(D)
    return sd


def rms(x, w, eps=1e-6):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def rope(x, pos, c):                                    # x [T, heads, Dh], half-split rotation
    inv = 1.0 / (c.rope_theta ** (torch.arange(0, c.head_dim, 2).float() / c.head_dim))
    ang = pos.float()[:, None] * inv[None]
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1)[:, None], torch.cat([ang.sin(), ang.sin()], -1)[:, None]
    half = x.shape[-1] // 2
    return x * cos + torch.cat([-x[..., half:], x[..., :half]], -1) * sin


def mot_forward(sd, c, seq, pos, text_idx, vae_idx, past, causal):
    """seq [T, D] packed query rows -> (final hidden [T, D], list of (k, v) of the query rows per layer)."""
    H, Hkv, Dh = c.num_attention_heads, c.num_key_value_heads, c.head_dim
    x, new_kv = seq, []
    sfx_of = torch.zeros(seq.shape[0], dtype=torch.bool)
    sfx_of[vae_idx] = True

    def per_row(fn):                                        # apply the understanding / generation variant row-wise
        out = None
        for rows, sfx in ((text_idx, ""), (vae_idx, "_moe_gen")):
            if len(rows) == 0:
                continue
            y = fn(rows, sfx)
            if out is None:
                out = y.new_zeros((seq.shape[0],) + y.shape[1:])
            out[rows] = y
        return out
    for i in range(c.num_hidden_layers):
        p = f"language_model.model.layers.{i}."
        lin = lambda t, n, sfx: F.linear(t, sd[p + n.format(sfx) + ".weight"], sd.get(p + n.format(sfx) + ".bias"))
        h = per_row(lambda r, s: rms(x[r], sd[p + f"input_layernorm{s}.weight"]))
        q = per_row(lambda r, s: rms(lin(h[r], "self_attn.q_proj{}", s).view(-1, H, Dh), sd[p + f"self_attn.q_norm{s}.weight"]))
        k = per_row(lambda r, s: rms(lin(h[r], "self_attn.k_proj{}", s).view(-1, Hkv, Dh), sd[p + f"self_attn.k_norm{s}.weight"]))
        v = per_row(lambda r, s: lin(h[r], "self_attn.v_proj{}", s).view(-1, Hkv, Dh))
        q, k = rope(q, pos, c), rope(k, pos, c)
        new_kv.append((k, v))
        kk, vv = (torch.cat([past[i][0], k]), torch.cat([past[i][1], v])) if past is not None else (k, v)
        kk, vv = kk.repeat_interleave(H // Hkv, 1), vv.repeat_interleave(H // Hkv, 1)
        s = torch.einsum("qhd,khd->hqk", q, kk) / math.sqrt(Dh)
        if causal:
            qi = torch.arange(q.shape[0])[:, None] + (kk.shape[0] - q.shape[0])
            s = s.masked_fill((torch.arange(kk.shape[0])[None] > qi)[None], float("-inf"))
        o = torch.einsum("hqk,khd->qhd", s.softmax(-1), vv).reshape(-1, H * Dh)
        x = x + per_row(lambda r, s_: lin(o[r], "self_attn.o_proj{}", s_))
        h = per_row(lambda r, s_: rms(x[r], sd[p + f"post_attention_layernorm{s_}.weight"]))
        x = x + per_row(lambda r, s_: lin(F.silu(lin(h[r], "mlp{}.gate_proj", s_)) * lin(h[r], "mlp{}.up_proj", s_), "mlp{}.down_proj", s_))
    final = per_row(lambda r, s_: rms(x[r], sd["language_model.model.norm" + s_ + ".weight"]))
    return final, new_kv


def flow_oracle(sd, c, x_t, t, h, w, past, position):
    N = h * w
    emb = sd["language_model.model.embed_tokens.weight"]
    seq = torch.zeros(N + 2, c.hidden_size)
    text_idx, vae_idx = torch.tensor([0, N + 1]), torch.arange(1, N + 1)
    seq[text_idx] = emb[[c.start_of_image, c.end_of_image]]
    half = 128
    args = t * torch.exp(-math.log(10000) * torch.arange(half).float() / half)
    tf = torch.cat([args.cos(), args.sin()])[None]
    temb = F.linear(F.silu(F.linear(tf, sd["time_embedder.mlp.0.weight"], sd["time_embedder.mlp.0.bias"])),
                    sd["time_embedder.mlp.2.weight"], sd["time_embedder.mlp.2.bias"])
    pos_ids = (torch.arange(h)[:, None] * c.max_latent_size + torch.arange(w)).flatten()
    seq[vae_idx] = F.linear(x_t, sd["vae2llm.weight"], sd["vae2llm.bias"]) + temb + sd["latent_pos_embed.pos_embed"][pos_ids]
    final, _ = mot_forward(sd, c, seq, torch.full((N + 2,), position), text_idx, vae_idx, past, causal=False)
    return F.linear(final, sd["llm2vae.weight"], sd["llm2vae.bias"])[vae_idx]


@pytest.fixture(scope="module")
def pair():
    torch.manual_seed(0)
    sd = _checkpoint(CFG)
    m = BagelMoT(CFG, torch.float32, "cpu")
    loaded = m.load_weights(sd.items())
    assert loaded == set(sd) - {"language_model.lm_head.weight", "connector.fc1.weight"}
    return sd, m


def test_understanding_prefill_and_generation_flow_match_the_oracle(pair):
    sd, m = pair
    c = CFG
    ids = torch.tensor([c.bos_token_id, 5, 9, 11, 3, c.eos_token_id])
    emb = sd["language_model.model.embed_tokens.weight"]
    with torch.no_grad():
        _, ref_kv = mot_forward(sd, c, emb[ids], torch.arange(6), torch.arange(6), torch.tensor([], dtype=torch.long), None, causal=True)
        ctx = m.prefill_text(ids)
    for (rk, rv), (k, v) in zip(ref_kv, ctx):
        assert (rk - k).abs().max().item() < 1e-5 and (rv - v).abs().max().item() < 1e-5
    # a second turn appended to the context keeps positions running
    more = torch.tensor([c.bos_token_id, 7, c.eos_token_id])
    with torch.no_grad():
        _, ref2 = mot_forward(sd, c, emb[more], torch.arange(6, 9), torch.arange(3), torch.tensor([], dtype=torch.long), ref_kv, causal=True)
        ctx2 = m.prefill_text(more, ctx, start_position=6)
    assert ctx2[1][0].shape[0] == 9 and (ctx2[1][0][6:] - ref2[1][0]).abs().max().item() < 1e-5
    h, w = 3, 2
    x_t = torch.randn(h * w, c.patch_latent_dim)
    with torch.no_grad():
        ref = flow_oracle(sd, c, x_t, torch.tensor(0.7), h, w, ref_kv, 6)
        out = m.flow(x_t[None], torch.tensor([0.7]), (h, w), ctx, 6)[0]
        assert (ref - out).abs().max().item() < 2e-5 * max(1.0, ref.abs().max().item())
        ref0 = flow_oracle(sd, c, x_t, torch.tensor(0.2), h, w, None, 0)            # empty context (unconditional branch)
        out0 = m.flow(x_t[None], torch.tensor([0.2]), (h, w), None, 0)[0]
        assert (ref0 - out0).abs().max().item() < 2e-5 * max(1.0, ref0.abs().max().item())


def test_marker_rows_only_variant(pair):
    sd, m = pair
    import dataclasses
    m2 = BagelMoT(dataclasses.replace(CFG, keep_embedding_table=False), torch.float32, "cpu")
    m2.load_weights(sd.items())
    assert m2.embed_tokens.shape == (2, CFG.hidden_size)
    x = torch.randn(1, 4, CFG.patch_latent_dim)
    kv = m.prefill_text(torch.tensor([58, 4, 59]))
    with torch.no_grad():
        assert torch.allclose(m.flow(x, torch.tensor([0.5]), (2, 2), kv, 3), m2.flow(x, torch.tensor([0.5]), (2, 2), kv, 3), atol=1e-6)


def test_position_table_time_grid_and_guidance():
    tab = sincos_2d_table(16, 4)
    # column first: position (row 2, col 3) -> first half encodes 3, second half encodes 2
    om = 1.0 / 10000 ** (np.arange(4) / 4.0)
    want = np.concatenate([np.sin(3 * om), np.cos(3 * om), np.sin(2 * om), np.cos(2 * om)])
    assert np.allclose(tab[2 * 4 + 3].numpy(), want, atol=1e-6)
    assert latent_position_ids(2, 3, 8).tolist() == [0, 1, 2, 8, 9, 10]
    ts = shifted_time_grid(5, 3.0)
    lin = torch.linspace(1, 0, 5)
    assert torch.allclose(ts, 3 * lin / (1 + 2 * lin)) and ts[0] == 1 and ts[-1] == 0
    v, vn = torch.randn(6, 8), torch.randn(6, 8)
    mix = vn + 4.0 * (v - vn)
    g = guided_velocity(v, vn, None, 4.0, 1.0, 0.0, "global")
    assert torch.allclose(g, mix * (v.norm() / (mix.norm() + 1e-8)).clamp(max=1.0))
    g = guided_velocity(v, vn, None, 4.0, 1.0, 0.0, "channel")
    assert torch.allclose(g, mix * (v.norm(dim=-1, keepdim=True) / (mix.norm(dim=-1, keepdim=True) + 1e-8)).clamp(max=1.0))
    assert guided_velocity(v, vn, None, 1.0) is v


def test_bagel_stage_text_to_image_and_injected_context():
    from vllm_omni_b200.diffusion.data import OmniDiffusionConfig, TransformerConfig
    from vllm_omni_b200.diffusion.models.bagel.pipeline import BagelPipeline
    from vllm_omni_b200.diffusion.request import OmniDiffusionRequest
    from vllm_omni_b200.inputs import OmniDiffusionSamplingParams
    torch.manual_seed(1)
    tf = {k: getattr(CFG, k) for k in CFG.__dataclass_fields__}
    vae = dict(block_out_channels=(8, 16, 16, 16), layers_per_block=1, norm_num_groups=4)
    cfg = OmniDiffusionConfig(dtype=torch.float32, tf_model_config=TransformerConfig.from_dict(tf), vae_config=vae, output_type="latent")
    pipe = BagelPipeline(cfg, device="cpu")
    sp = lambda **kw: OmniDiffusionSamplingParams(height=64, width=32, num_inference_steps=4, seed=2, output_type="latent", **kw)
    run = lambda prompt, s: pipe(OmniDiffusionRequest(prompts=[prompt], sampling_params=s, request_ids=["r"])).output
    a = run("a cube", sp())
    assert a.shape == (1, 4, 8, 4) and torch.isfinite(a).all()
    b = run("a cube", sp(extra_args={"cfg_text_scale": 1.0}))
    assert not torch.allclose(a, b)                         # guidance against the empty prompt changes the sample
    # the context handed over as KV equals prefilling the same ids here (guidance is off on that path)
    ids = pipe._prompt_ids("a cube")
    s = sp()
    s.past_key_values = pipe.transformer.prefill_text(ids)
    c = run("ignored", s)
    assert torch.allclose(c, b, atol=1e-5)
    img = pipe(OmniDiffusionRequest(prompts=["a cube"], sampling_params=OmniDiffusionSamplingParams(height=32, width=32, num_inference_steps=2, seed=2,
                                                                                                   output_type="pt"), request_ids=["r"])).output
    assert img.shape[-2:] == (32, 32)


def test_ar_stage_cache_equals_the_generation_stage_prefill(pair):
    """The AR stage (understanding weights of the same checkpoint, ``llm_config`` geometry) fills a paged
    KV cache whose rows equal what the generation stage would prefill itself: the context it hands over
    is exactly the one the denoiser expects."""
    from vllm_omni_b200.models.local_decode import LocalDecodeSession
    from vllm_omni_b200.models.text import build_text_model
    sd, m = pair
    c = CFG
    hf = {"architectures": ["BagelForConditionalGeneration"],
          "llm_config": dict(vocab_size=c.vocab_size, hidden_size=c.hidden_size, num_hidden_layers=c.num_hidden_layers,
                             num_attention_heads=c.num_attention_heads, num_key_value_heads=c.num_key_value_heads,
                             intermediate_size=c.intermediate_size, rope_theta=c.rope_theta, rms_norm_eps=c.rms_norm_eps)}
    ar = build_text_model("thinker", hf, torch.float32, "cpu")
    loaded = ar.load_weights(sd.items())
    assert "model.layers.0.self_attn.q_norm.weight" in loaded and not any("moe_gen" in n for n in loaded)
    ids = torch.tensor([c.bos_token_id, 5, 9, 11, 3, c.eos_token_id])
    sess = LocalDecodeSession(ar.decoder, 32)
    sess.prefill(ids=ids)
    ctx = m.prefill_text(ids)
    for (kp, vp), (k, v) in zip(sess.caches, ctx):
        assert (kp.flatten(0, 1)[:6] - k).abs().max().item() < 1e-5 and (vp.flatten(0, 1)[:6] - v).abs().max().item() < 1e-5


def test_image_context_blocks_match_the_oracle(pair):
    """Editing context: clean VAE latents (generation weights, timestep 0) and vision tokens (understanding
    weights), each between the image markers at ONE rotary position with full attention, appended to the cache."""
    sd, m = pair
    c = CFG
    torch.manual_seed(3)
    h, w = 2, 3
    N = h * w
    lat = torch.randn(N, c.patch_latent_dim)
    ctx = m.prefill_image_latents(lat, (h, w), None, 0)
    # oracle: [start, latents..., end] at position 0, t = 0
    emb = sd["language_model.model.embed_tokens.weight"]
    seq = torch.zeros(N + 2, c.hidden_size)
    text_idx, vae_idx = torch.tensor([0, N + 1]), torch.arange(1, N + 1)
    seq[text_idx] = emb[[c.start_of_image, c.end_of_image]]
    tf = torch.cat([torch.ones(128), torch.zeros(128)])[None]            # sinusoid of t = 0: cosines first
    temb = F.linear(F.silu(F.linear(tf, sd["time_embedder.mlp.0.weight"], sd["time_embedder.mlp.0.bias"])),
                    sd["time_embedder.mlp.2.weight"], sd["time_embedder.mlp.2.bias"])
    pos_ids = (torch.arange(h)[:, None] * c.max_latent_size + torch.arange(w)).flatten()
    seq[vae_idx] = F.linear(lat, sd["vae2llm.weight"], sd["vae2llm.bias"]) + temb + sd["latent_pos_embed.pos_embed"][pos_ids]
    _, kv = mot_forward(sd, c, seq, torch.zeros(N + 2, dtype=torch.long), text_idx, vae_idx, None, causal=False)
    order = torch.cat([vae_idx, text_idx])                               # this build keeps the latent rows first
    for (k, v), (ko, vo) in zip(ctx, kv):
        assert k.shape[0] == N + 2 and torch.allclose(k, ko[order], atol=1e-5) and torch.allclose(v, vo[order], atol=1e-5)
    # vision tokens after it, at position 1, against the grown context
    vt = torch.randn(5, c.hidden_size)
    ctx2 = m.prefill_vision_tokens(vt, ctx, 1)
    seq2 = torch.cat([emb[[c.start_of_image]], vt, emb[[c.end_of_image]]])
    past = [(ko[order], vo[order]) for ko, vo in kv]
    _, kv2 = mot_forward(sd, c, seq2, torch.ones(7, dtype=torch.long), torch.arange(7), torch.tensor([], dtype=torch.long), past, causal=False)
    order2 = torch.tensor([1, 2, 3, 4, 5, 0, 6])
    for (k, v), (ko, vo) in zip(ctx2, kv2):
        assert k.shape[0] == N + 2 + 7 and torch.allclose(k[N + 2:], ko[order2], atol=1e-5) and torch.allclose(v[N + 2:], vo[order2], atol=1e-5)
    # the prompt follows causally from position 2
    ids = torch.tensor([c.bos_token_id, 5, 9, c.eos_token_id])
    ctx3 = m.prefill_text(ids, ctx2, 2)
    assert ctx3[0][0].shape[0] == N + 2 + 7 + 4


def test_vision_tower_matches_hf_siglip_encoder():
    from transformers import SiglipVisionConfig, SiglipVisionModel
    from vllm_omni_b200.diffusion.models.bagel.vision import BagelVisionTower, BagelVitConfig, flat_position_ids, patchify_pixels
    torch.manual_seed(4)
    hf_cfg = SiglipVisionConfig(hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4, patch_size=4,
                                image_size=24, hidden_act="gelu_pytorch_tanh", layer_norm_eps=1e-6)
    hf = SiglipVisionModel(hf_cfg).eval()
    vc = BagelVitConfig(hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4, patch_size=4,
                        max_patches_per_side=6)
    tower = BagelVisionTower(vc, llm_width=40, dtype=torch.float32, device="cpu")
    sd = {"vit_model." + k: v for k, v in hf.state_dict().items()}
    sd["connector.fc1.weight"], sd["connector.fc1.bias"] = torch.randn(40, 32) * 0.1, torch.randn(40) * 0.1
    sd["connector.fc2.weight"], sd["connector.fc2.bias"] = torch.randn(40, 40) * 0.1, torch.randn(40) * 0.1
    loaded = tower.load_weights(sd.items())
    skipped = {k for k in sd if k not in loaded}
    assert all("post_layernorm" in k or ".head." in k for k in skipped), skipped     # the encoder output is used as is
    px = torch.rand(3, 12, 20) * 2 - 1                                     # 3 x 5 patches, native aspect ratio
    got = tower(px)
    with torch.no_grad():
        ids = flat_position_ids(3, 5, 6)
        w = hf.vision_model.embeddings.patch_embedding.weight
        x = F.linear(patchify_pixels(px, 4), w.view(w.shape[0], -1), hf.vision_model.embeddings.patch_embedding.bias)
        x = x + hf.vision_model.embeddings.position_embedding(ids)
        y = hf.vision_model.encoder(inputs_embeds=x[None]).last_hidden_state[0]
        want = F.linear(F.gelu(F.linear(y, sd["connector.fc1.weight"], sd["connector.fc1.bias"]), approximate="tanh"),
                        sd["connector.fc2.weight"], sd["connector.fc2.bias"]) + tower.vit_pos_embed[ids]
    assert got.shape == (15, 40) and (got - want).abs().max() < 1e-4


def test_bagel_stage_edits_a_reference_image():
    import numpy as np
    from PIL import Image
    from vllm_omni_b200.diffusion.data import OmniDiffusionConfig, TransformerConfig
    from vllm_omni_b200.diffusion.models.bagel.pipeline import BagelPipeline
    from vllm_omni_b200.diffusion.request import OmniDiffusionRequest
    from vllm_omni_b200.inputs import OmniDiffusionSamplingParams
    torch.manual_seed(1)
    tf = {k: getattr(CFG, k) for k in CFG.__dataclass_fields__}
    tf["max_latent_size"] = 32
    tf["vit_config"] = dict(hidden_size=32, intermediate_size=48, num_hidden_layers=1, num_attention_heads=4, patch_size=14)
    vae = dict(block_out_channels=(8, 16, 16, 16), layers_per_block=1, norm_num_groups=4)
    cfg = OmniDiffusionConfig(dtype=torch.float32, tf_model_config=TransformerConfig.from_dict(tf), vae_config=vae, output_type="latent")
    pipe = BagelPipeline(cfg, device="cpu")
    rng = np.random.default_rng(0)
    imgs = [Image.fromarray(rng.integers(0, 255, (250, 300, 3), dtype=np.uint8)) for _ in range(2)]
    assert pipe._fit_reference(imgs[0], 512, 16).size == (304, 256)        # shortest side up to 256, both multiples of 16

    def run(img, **extra):
        sp = OmniDiffusionSamplingParams(num_inference_steps=3, seed=2, output_type="latent", extra_args=extra or None)
        req = OmniDiffusionRequest(prompts=[{"prompt": "make it red", "multi_modal_data": {"image": img}}], sampling_params=sp,
                                   request_ids=["r"])
        return pipe(req).output
    a, b = run(imgs[0]), run(imgs[1])
    assert a.shape == (1, 4, 32, 38) and torch.isfinite(a).all()           # the result has the reference image's (fitted) size
    assert (a - b).abs().max() > 0                                         # the image reaches the network
    assert (a - run(imgs[0], cfg_img_scale=1.0)).abs().max() > 0           # and so does the image-guidance branch
    ctx, pos = pipe._image_context(pipe._fit_reference(imgs[0], 512, 16))
    n_lat, n_vit = (256 // 16) * (304 // 16), (256 // 14) * (304 // 14)
    assert pos == 2 and ctx[0][0].shape[0] == n_lat + 2 + n_vit + 2
