"""Stable Audio: the DiT against a straight-line restatement of the published architecture on a dict
of diffusers-named tensors, the projection model, the Oobleck autoencoder against torch modules with
``weight_norm`` built in the test, and the SDE DPM-Solver++ sampler against its closed-form steps."""
import math

import torch
import torch.nn.functional as F
from torch import nn

from vllm_omni_b200.diffusion.models.stable_audio.transformer import (StableAudioDiTConfig, StableAudioDiTModel,
                                                                      StableAudioProjectionConfig, StableAudioProjectionModel)
from vllm_omni_b200.diffusion.models.vae.oobleck import AutoencoderOobleck, OobleckConfig
from vllm_omni_b200.diffusion.schedulers.cosine_dpm import CosineDPMSolverMultistepScheduler

CFG = StableAudioDiTConfig(sample_size=12, in_channels=8, num_layers=2, attention_head_dim=16, num_attention_heads=4,
                           num_key_value_attention_heads=2, out_channels=8, cross_attention_dim=24, time_proj_dim=16,
                           global_states_input_dim=40, cross_attention_input_dim=20)


def _names(c):
    D, kv, Fi = c.num_attention_heads * c.attention_head_dim, c.num_key_value_attention_heads * c.attention_head_dim, 4 * c.num_attention_heads * c.attention_head_dim
    sd = {"time_proj.weight": (c.time_proj_dim // 2,), "timestep_proj.0.weight": (D, c.time_proj_dim), "timestep_proj.0.bias": (D,),
          "timestep_proj.2.weight": (D, D), "timestep_proj.2.bias": (D,), "global_proj.0.weight": (D, c.global_states_input_dim),
          "global_proj.2.weight": (D, D), "cross_attention_proj.0.weight": (c.cross_attention_dim, c.cross_attention_input_dim),
          "cross_attention_proj.2.weight": (c.cross_attention_dim, c.cross_attention_dim),
          "preprocess_conv.weight": (c.in_channels, c.in_channels, 1), "postprocess_conv.weight": (c.out_channels, c.out_channels, 1),
          "proj_in.weight": (D, c.in_channels), "proj_out.weight": (c.out_channels, D)}
    for i in range(c.num_layers):
        b = f"transformer_blocks.{i}."
        for n in ("norm1", "norm2", "norm3"):
            sd[b + n + ".weight"], sd[b + n + ".bias"] = (D,), (D,)
        for n in ("to_q", "to_k", "to_v", "to_out.0"):
            sd[b + f"attn1.{n}.weight"] = (D, D)
        sd[b + "attn2.to_q.weight"], sd[b + "attn2.to_out.0.weight"] = (D, D), (D, D)
        sd[b + "attn2.to_k.weight"], sd[b + "attn2.to_v.weight"] = (kv, c.cross_attention_dim), (kv, c.cross_attention_dim)
        sd[b + "ff.net.0.proj.weight"], sd[b + "ff.net.0.proj.bias"] = (2 * Fi, D), (2 * Fi,)
        sd[b + "ff.net.2.weight"], sd[b + "ff.net.2.bias"] = (D, Fi), (D,)
    return sd


def dit_oracle(sd, c, lat, t, enc, glob):
    H, Hkv, Dh = c.num_attention_heads, c.num_key_value_attention_heads, c.attention_head_dim
    lin = lambda x, n: F.linear(x, sd[n + ".weight"], sd.get(n + ".bias"))
    ctx = lin(F.silu(lin(enc, "cross_attention_proj.0")), "cross_attention_proj.2")
    g = lin(F.silu(lin(glob, "global_proj.0")), "global_proj.2")
    proj = 2 * math.pi * t[:, None] @ sd["time_proj.weight"][None, :]
    temb = lin(F.silu(lin(torch.cat([proj.cos(), proj.sin()], -1), "timestep_proj.0")), "timestep_proj.2")
    g = g + temb.unsqueeze(1)
    x = F.conv1d(lat, sd["preprocess_conv.weight"]) + lat
    x = lin(x.transpose(1, 2), "proj_in")
    x = torch.cat([g, x], 1)
    B, S, D = x.shape
    rd = Dh // 2
    freqs = 1.0 / (10000 ** (torch.arange(0, rd, 2)[: rd // 2].float() / rd))
    ang = torch.outer(torch.arange(S).float(), freqs)
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)

    def rope(h):                                            # [B, S, H, Dh]
        r, p = h[..., :rd], h[..., rd:]
        real, imag = r.reshape(*r.shape[:-1], 2, rd // 2).unbind(-2)
        rot = torch.cat([-imag, real], -1)
        return torch.cat([r * cos[None, :, None] + rot * sin[None, :, None], p], -1)

    def sdpa(q, k, v):
        return F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2).reshape(B, S, D)
    for i in range(c.num_layers):
        b = f"transformer_blocks.{i}."
        h = F.layer_norm(x, (D,), sd[b + "norm1.weight"], sd[b + "norm1.bias"])
        q, k, v = (lin(h, b + f"attn1.{n}").view(B, S, H, Dh) for n in ("to_q", "to_k", "to_v"))
        x = x + lin(sdpa(rope(q), rope(k), v), b + "attn1.to_out.0")
        h = F.layer_norm(x, (D,), sd[b + "norm2.weight"], sd[b + "norm2.bias"])
        q = lin(h, b + "attn2.to_q").view(B, S, H, Dh)
        k, v = (lin(ctx, b + f"attn2.{n}").view(B, -1, Hkv, Dh).repeat_interleave(H // Hkv, dim=2) for n in ("to_k", "to_v"))
        x = x + lin(sdpa(q, k, v), b + "attn2.to_out.0")
        h = F.layer_norm(x, (D,), sd[b + "norm3.weight"], sd[b + "norm3.bias"])
        val, gate = lin(h, b + "ff.net.0.proj").chunk(2, -1)
        x = x + lin(val * F.silu(gate), b + "ff.net.2")
    y = lin(x, "proj_out").transpose(1, 2)[:, :, 1:]
    return F.conv1d(y, sd["postprocess_conv.weight"]) + y


def test_dit_forward_from_diffusers_named_tensors():
    torch.manual_seed(0)
    sd = {n: torch.randn(s) * (0.1 if len(s) > 1 else 0.2) + (1.0 if "norm" in n and n.endswith("weight") else 0.0)
          for n, s in _names(CFG).items()}
    m = StableAudioDiTModel(CFG, torch.float32, "cpu")
    assert m.load_weights(sd.items()) == set(sd)
    B, L, S = 2, 12, 7
    lat, t = torch.randn(B, 8, L), torch.tensor([0.8, 0.8])
    enc, glob = torch.randn(B, S, 20), torch.randn(B, 1, 40)
    with torch.no_grad():
        ref = dit_oracle(sd, CFG, lat, t, enc, glob)
        out = m(lat, t[:1], encoder_hidden_states=enc, global_hidden_states=glob)
        kv = m.conditioning(enc)                            # cached keys / values give the same result
        out2 = m(lat, t, global_hidden_states=glob, cross_kv=kv)
    assert out.shape == ref.shape == (B, 8, L)
    assert (out - ref).abs().max().item() < 2e-4 * max(1.0, ref.abs().max().item())
    assert torch.equal(out, out2)


def test_projection_model_number_conditioners():
    torch.manual_seed(1)
    pm = StableAudioProjectionModel(StableAudioProjectionConfig(text_encoder_dim=20, conditioning_dim=24, min_value=0, max_value=512),
                                    torch.float32, "cpu")
    sd = {"text_projection.weight": torch.randn(24, 20), "text_projection.bias": torch.randn(24)}
    for c in ("start_number_conditioner", "end_number_conditioner"):
        sd[c + ".time_positional_embedding.0.weights"] = torch.randn(128)
        sd[c + ".time_positional_embedding.1.weight"] = torch.randn(24, 257) * 0.1
        sd[c + ".time_positional_embedding.1.bias"] = torch.randn(24)
    assert pm.load_weights(sd.items()) == set(sd)
    sec = torch.tensor([0.0, 30.0, 600.0])
    x = (sec.clamp(0, 512) / 512)[:, None]
    f = x * sd["end_number_conditioner.time_positional_embedding.0.weights"][None] * 2 * math.pi
    ref = F.linear(torch.cat([x, f.sin(), f.cos()], -1), sd["end_number_conditioner.time_positional_embedding.1.weight"],
                   sd["end_number_conditioner.time_positional_embedding.1.bias"])
    out = pm.end_number_conditioner(sec)
    assert out.shape == (3, 1, 24) and (out[:, 0] - ref).abs().max().item() < 1e-5
    st = torch.randn(2, 5, 20)
    assert (pm.project_text(st) - F.linear(st, sd["text_projection.weight"], sd["text_projection.bias"])).abs().max().item() < 1e-5


# ----------------------------------------------------------------------------- Oobleck
def _wn(m):
    return nn.utils.weight_norm(m)


class _Snake(nn.Module):
    def __init__(self, ch):
        super().__init__()
        self.alpha, self.beta = nn.Parameter(torch.randn(1, ch, 1) * 0.3), nn.Parameter(torch.randn(1, ch, 1) * 0.3)

    def forward(self, x):
        return x + (self.beta.exp() + 1e-9).reciprocal() * torch.sin(self.alpha.exp() * x).pow(2)


class _Res(nn.Module):
    def __init__(self, ch, d):
        super().__init__()
        self.snake1, self.conv1 = _Snake(ch), _wn(nn.Conv1d(ch, ch, 7, dilation=d, padding=((7 - 1) * d) // 2))
        self.snake2, self.conv2 = _Snake(ch), _wn(nn.Conv1d(ch, ch, 1))

    def forward(self, x):
        return x + self.conv2(self.snake2(self.conv1(self.snake1(x))))


class _DecBlock(nn.Module):
    def __init__(self, cin, cout, s):
        super().__init__()
        self.snake1 = _Snake(cin)
        self.conv_t1 = _wn(nn.ConvTranspose1d(cin, cout, 2 * s, stride=s, padding=math.ceil(s / 2)))
        self.res_unit1, self.res_unit2, self.res_unit3 = _Res(cout, 1), _Res(cout, 3), _Res(cout, 9)

    def forward(self, x):
        return self.res_unit3(self.res_unit2(self.res_unit1(self.conv_t1(self.snake1(x)))))


class _EncBlock(nn.Module):
    def __init__(self, cin, cout, s):
        super().__init__()
        self.res_unit1, self.res_unit2, self.res_unit3 = _Res(cin, 1), _Res(cin, 3), _Res(cin, 9)
        self.snake1 = _Snake(cin)
        self.conv1 = _wn(nn.Conv1d(cin, cout, 2 * s, stride=s, padding=math.ceil(s / 2)))

    def forward(self, x):
        return self.conv1(self.snake1(self.res_unit3(self.res_unit2(self.res_unit1(x)))))


class _OobleckOracle(nn.Module):
    def __init__(self, c: OobleckConfig):
        super().__init__()
        mult, ch = (1,) + tuple(c.channel_multiples), c.decoder_channels
        strides = c.downsampling_ratios[::-1]
        n = len(strides)
        dec = nn.Module()
        dec.conv1 = _wn(nn.Conv1d(c.decoder_input_channels, ch * mult[-1], 7, padding=3))
        dec.block = nn.ModuleList([_DecBlock(ch * mult[n - i], ch * mult[n - i - 1], s) for i, s in enumerate(strides)])
        dec.snake1 = _Snake(ch)
        dec.conv2 = _wn(nn.Conv1d(ch, c.audio_channels, 7, padding=3, bias=False))
        enc = nn.Module()
        eh = c.encoder_hidden_size
        enc.conv1 = _wn(nn.Conv1d(c.audio_channels, eh, 7, padding=3))
        enc.block = nn.ModuleList([_EncBlock(eh * mult[i], eh * mult[i + 1], s) for i, s in enumerate(c.downsampling_ratios)])
        enc.snake1 = _Snake(eh * mult[-1])
        enc.conv2 = _wn(nn.Conv1d(eh * mult[-1], eh, 3, padding=1))
        self.decoder, self.encoder = dec, enc

    @staticmethod
    def run(part, x):
        x = part.conv1(x)
        for b in part.block:
            x = b(x)
        return part.conv2(part.snake1(x))


def test_oobleck_against_weight_normed_torch_modules():
    torch.manual_seed(2)
    c = OobleckConfig(encoder_hidden_size=8, downsampling_ratios=(2, 4), channel_multiples=(1, 2), decoder_channels=6,
                      decoder_input_channels=4, audio_channels=2)
    o = _OobleckOracle(c).eval()
    with torch.no_grad():
        for n, p in o.named_parameters():                   # weight-norm gains away from the norm of v
            if n.endswith(("weight_g", "original0")):
                p.mul_(torch.rand_like(p) + 0.5)
    m = AutoencoderOobleck(c, torch.float32, "cpu", with_encoder=True)
    sd = o.state_dict()
    assert any(k.endswith(("weight_g", "parametrizations.weight.original0")) for k in sd)
    loaded = m.load_weights(sd.items())
    assert loaded == set(sd), sorted(set(sd) - loaded)
    z, wav = torch.randn(2, 4, 9), torch.randn(2, 2, 64)
    with torch.no_grad():
        ref, out = o.run(o.decoder, z), m.decode(z)
        assert out.shape == ref.shape == (2, 2, 9 * 8) and (out - ref).abs().max().item() < 1e-5
        ref = o.run(o.encoder, wav)
        mean = m.encode(wav, sample=False)
        assert mean.shape == (2, 4, 8) and (mean - ref[:, :4]).abs().max().item() < 1e-5
        g = torch.Generator().manual_seed(3)
        z = m.encode(wav, generator=g)
        std = F.softplus(ref[:, 4:]) + 1e-4
        g = torch.Generator().manual_seed(3)
        assert (z - (ref[:, :4] + std * torch.randn(mean.shape, generator=g))).abs().max().item() < 1e-5


# ----------------------------------------------------------------------------- sampler
def test_sde_dpm_solver_steps_follow_the_closed_form():
    s = CosineDPMSolverMultistepScheduler()
    ts = s.set_timesteps(6)
    sig = s.sigmas
    assert abs(float(sig[0]) - 500) < 1e-6 and abs(float(sig[5]) - 0.3) < 1e-9 and float(sig[6]) == 0.0
    assert torch.allclose(ts.double(), torch.atan(sig[:-1]) * 2 / math.pi, atol=1e-6)
    assert abs(s.init_noise_sigma - math.sqrt(500 ** 2 + 1)) < 1e-9
    torch.manual_seed(0)
    x = torch.randn(2, 3, 5) * s.init_noise_sigma
    outs, noises, xs = [], [], [x]
    for i in range(6):
        xin = s.scale_model_input(xs[-1])
        assert torch.allclose(xin, xs[-1] / math.sqrt(float(sig[i]) ** 2 + 1), atol=1e-6)
        v = torch.randn(2, 3, 5)
        z = torch.randn(2, 3, 5)
        outs.append(v), noises.append(z)
        xs.append(s.step(v, xs[-1], noise=z))
    # restate: x0 estimates, then first / second order updates
    x0 = []
    for i in range(6):
        si = float(sig[i])
        x0.append(xs[i] / (si * si + 1) - si / math.sqrt(si * si + 1) * outs[i])
    lam = lambda v: -math.log(v)
    s0, s1 = float(sig[0]), float(sig[1])
    h = lam(s1) - lam(s0)
    want = s1 / s0 * math.exp(-h) * xs[0] + (1 - math.exp(-2 * h)) * x0[0] + s1 * math.sqrt(1 - math.exp(-2 * h)) * noises[0]
    assert torch.allclose(xs[1], want, rtol=1e-5, atol=1e-4)
    i = 3
    st, s0, sp = float(sig[i + 1]), float(sig[i]), float(sig[i - 1])
    h, h0 = lam(st) - lam(s0), lam(s0) - lam(sp)
    d1 = (x0[i] - x0[i - 1]) / (h0 / h)
    want = (st / s0 * math.exp(-h)) * xs[i] + (1 - math.exp(-2 * h)) * x0[i] + 0.5 * (1 - math.exp(-2 * h)) * d1 \
        + st * math.sqrt(1 - math.exp(-2 * h)) * noises[i]
    assert torch.allclose(xs[i + 1], want, rtol=1e-5, atol=1e-4)
    assert torch.allclose(xs[6], x0[5], atol=1e-6)          # the last step lands on the clean estimate


def test_sampler_recovers_a_point_mass():
    """With the exact v-prediction of a data distribution concentrated on one point x*, every clean
    estimate is x*, so the sampler returns x* whatever noise it injects."""
    s = CosineDPMSolverMultistepScheduler()
    s.set_timesteps(8)
    target = torch.tensor([[[0.3, -0.7, 1.1]]])
    x = torch.randn(1, 1, 3) * s.init_noise_sigma
    for i in range(8):
        sg = float(s.sigmas[i])
        # v with c_skip x + c_out v = x*  ->  v = (c_skip x - x*) / (sigma / sqrt(sigma^2 + 1))
        v = (x / (sg * sg + 1) - target) / (sg / math.sqrt(sg * sg + 1))
        x = s.step(v, x)
    assert torch.allclose(x, target, atol=1e-4)


def test_stable_audio_folder_through_the_loader(tmp_path):
    """A diffusers-layout folder (transformer/, vae/ with weight-norm pairs, projection_model/, scheduler/,
    text_encoder/ = T5, tokenizer/) is loaded by name and generates a stereo clip of the asked length."""
    import json

    import pytest
    transformers = pytest.importorskip("transformers")
    pytest.importorskip("tokenizers")
    from test_text_encoders import _init, _tokenizer_dir
    from vllm_omni_b200.diffusion.loader import DiffusersPipelineLoader
    from vllm_omni_b200.diffusion.request import OmniDiffusionRequest
    from vllm_omni_b200.entrypoints.omni_diffusion import build_diffusion_config
    from vllm_omni_b200.inputs import OmniDiffusionSamplingParams
    from vllm_omni_b200.utils.safetensors_reader import save_safetensors
    torch.manual_seed(0)
    d = tmp_path
    (d / "model_index.json").write_text(json.dumps({"_class_name": "StableAudioPipeline"}))
    for sub in ("transformer", "vae", "projection_model", "scheduler"):
        (d / sub).mkdir()
    tc = {k: getattr(CFG, k) for k in CFG.__dataclass_fields__}
    (d / "transformer" / "config.json").write_text(json.dumps({"_class_name": "StableAudioDiTModel", **tc}))
    sd = {n: torch.randn(s) * (0.1 if len(s) > 1 else 0.2) + (1.0 if "norm" in n and n.endswith("weight") else 0.0)
          for n, s in _names(CFG).items()}
    save_safetensors(sd, str(d / "transformer" / "diffusion_pytorch_model.safetensors"))
    oc = OobleckConfig(encoder_hidden_size=8, downsampling_ratios=(2, 4), channel_multiples=(1, 2), decoder_channels=6,
                       decoder_input_channels=8, audio_channels=2, sampling_rate=800)
    (d / "vae" / "config.json").write_text(json.dumps({k: (list(v) if isinstance(v, tuple) else v) for k, v in oc.__dict__.items()}))
    vo = _OobleckOracle(oc).eval()
    save_safetensors({k: v.detach().clone().contiguous() for k, v in vo.state_dict().items()}, str(d / "vae" / "diffusion_pytorch_model.safetensors"))
    (d / "projection_model" / "config.json").write_text(json.dumps(dict(text_encoder_dim=20, conditioning_dim=20, min_value=0, max_value=512)))
    psd = {}
    for c in ("start_number_conditioner", "end_number_conditioner"):
        psd[c + ".time_positional_embedding.0.weights"] = torch.randn(128)
        psd[c + ".time_positional_embedding.1.weight"] = torch.randn(20, 257) * 0.1
        psd[c + ".time_positional_embedding.1.bias"] = torch.randn(20)
    save_safetensors(psd, str(d / "projection_model" / "diffusion_pytorch_model.safetensors"))
    (d / "scheduler" / "scheduler_config.json").write_text(json.dumps(dict(_class_name="CosineDPMSolverMultistepScheduler", sigma_min=0.3,
                                                                            sigma_max=500, sigma_data=1.0, solver_order=2,
                                                                            prediction_type="v_prediction", sigma_schedule="exponential")))
    hc = transformers.T5Config(vocab_size=40, d_model=20, d_kv=5, d_ff=32, num_layers=2, num_heads=2,
                               relative_attention_num_buckets=8, relative_attention_max_distance=16, feed_forward_proj="relu")
    t5 = _init(transformers.T5EncoderModel(hc))
    t5.save_pretrained(str(d / "text_encoder"))
    _tokenizer_dir(d / "tokenizer", 16)
    cfg = build_diffusion_config(str(d), dtype="float32")
    pipe = DiffusersPipelineLoader(cfg).load_model("cpu")
    assert torch.equal(pipe.transformer.proj_in.weight, sd["proj_in.weight"])
    assert torch.equal(pipe.projection_model.end_number_conditioner.weights, psd["end_number_conditioner.time_positional_embedding.0.weights"])
    assert pipe.vae.hop_length == 8 and pipe.scheduler.config["sigma_max"] == 500
    z = torch.randn(1, 8, 5)
    with torch.no_grad():
        assert (pipe.vae.decode(z) - vo.run(vo.decoder, z)).abs().max().item() < 1e-5
        tok = transformers.AutoTokenizer.from_pretrained(str(d / "tokenizer"))
        enc = tok(["a red cube on the table"], padding="max_length", max_length=16, truncation=True, return_tensors="pt")
        ref = t5(enc.input_ids, attention_mask=enc.attention_mask).last_hidden_state * enc.attention_mask[..., None]
        got = pipe.encode_prompt(["a red cube on the table"])
        assert got.shape == (1, 16, 20) and (got - ref).abs().max().item() < 2e-5 * max(1.0, ref.abs().max().item())
        assert (got[0, enc.attention_mask[0] == 0] == 0).all() and enc.attention_mask.sum() < 16
    sp = OmniDiffusionSamplingParams(num_inference_steps=3, seed=1, guidance_scale=3.0,
                                     extra_args={"audio_start_in_s": 0.01, "audio_end_in_s": 0.11})
    out = pipe(OmniDiffusionRequest(prompts=[{"prompt": "a red cube", "negative_prompt": "blurry"}], sampling_params=sp, request_ids=["r"]))
    wav = out.output[0]
    assert wav.shape == (2, 88 - 8) and torch.isfinite(wav).all() and out.metrics["sample_rate"] == 800
