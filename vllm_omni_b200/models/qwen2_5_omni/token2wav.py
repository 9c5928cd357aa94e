"""Qwen2.5-Omni token2wav ("code2wav" stage): codec tokens -> mel spectrogram by a flow-matching
DiT integrated with a Runge-Kutta (3/8 rule) solver under classifier-free guidance, then a
BigVGAN-style vocoder mel -> 24 kHz waveform
(vllm_omni/model_executor/models/qwen2_5_omni/qwen2_5_omni_token2wav.py:385-1860).

DiT: codec embedding repeated ``repeats`` times per token, concatenated with the noisy mel and
a conditioning (speaker) vector, AdaLN-zero blocks with rotary attention restricted to a band
of blocks (``look_backward_blocks`` / ``look_ahead_blocks`` of ``block_size`` frames), which is
what makes chunked streaming decode possible.  Sampling: x(0) ~ N(0, 1), time grid
``linspace(0, 1, num_steps)`` warped by ``t + s (cos(pi t / 2) - 1 + t)``, velocity
``v = v_cond + g (v_cond - v_null)``.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from ..base import StageModel
from .config import BigVGANConfig, DiTConfig, Qwen25OmniConfig


def rk4_38_integrate(fn, x0: torch.Tensor, times: torch.Tensor) -> torch.Tensor:
    """Integrate dx/dt = fn(t, x) over the grid ``times`` with the 3/8-rule Runge-Kutta step."""
    x = x0
    for t0, t1 in zip(times[:-1], times[1:]):
        h = t1 - t0
        k1 = fn(t0, x)
        k2 = fn(t0 + h / 3, x + h * k1 / 3)
        k3 = fn(t0 + 2 * h / 3, x + h * (k2 - k1 / 3))
        k4 = fn(t1, x + h * (k1 - k2 + k3))
        x = x + (k1 + 3 * (k2 + k3) + k4) * h / 8
    return x


def sway_time_grid(num_steps: int, sway: float | None, device) -> torch.Tensor:
    t = torch.linspace(0, 1, num_steps, device=device)
    if sway is not None:
        t = t + sway * (torch.cos(math.pi / 2 * t) - 1 + t)
    return t


class _AdaLNZero(nn.Module):
    def __init__(self, dim, n, **kw):
        super().__init__()
        self.lin = nn.Linear(dim, n * dim, **kw)
        self.n = n

    def forward(self, emb):
        return self.lin(F.silu(emb)).chunk(self.n, dim=-1)


class DiTBlock(nn.Module):
    def __init__(self, c: DiTConfig, **kw):
        super().__init__()
        D, H, Dh = c.hidden_size, c.num_attention_heads, c.head_dim
        self.H, self.Dh = H, Dh
        self.mod = _AdaLNZero(D, 6, **kw)
        self.qkv = nn.Linear(D, 3 * H * Dh, **kw)
        self.out = nn.Linear(H * Dh, D, **kw)
        self.ff1 = nn.Linear(D, c.ff_mult * D, **kw)
        self.ff2 = nn.Linear(c.ff_mult * D, D, **kw)

    def forward(self, x, emb, cos, sin, mask):
        B, T, D = x.shape
        s1, c1, g1, s2, c2, g2 = self.mod(emb)
        h = F.layer_norm(x, (D,)) * (1 + c1[:, None]) + s1[:, None]
        q, k, v = self.qkv(h).view(B, T, 3, self.H, self.Dh).permute(2, 0, 3, 1, 4)
        q, k = _rope(q, cos, sin), _rope(k, cos, sin)
        a = F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
        x = x + g1[:, None] * self.out(a.transpose(1, 2).reshape(B, T, -1))
        h = F.layer_norm(x, (D,)) * (1 + c2[:, None]) + s2[:, None]
        return x + g2[:, None] * self.ff2(F.gelu(self.ff1(h), approximate="tanh"))


def _rope(x, cos, sin):
    x1, x2 = x[..., ::2], x[..., 1::2]
    return torch.stack([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1).flatten(-2)


class Token2WavDiT(nn.Module):
    def __init__(self, c: DiTConfig, dtype, device):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.c = c
        D = c.hidden_size
        self.codec_embed = nn.Embedding(c.num_embeds, c.emb_dim, **kw)
        self.in_proj = nn.Linear(c.mel_dim + c.emb_dim + c.speaker_dim, D, **kw)
        self.time_mlp = nn.Sequential(nn.Linear(256, D, **kw), nn.SiLU(), nn.Linear(D, D, **kw))
        self.blocks = nn.ModuleList([DiTBlock(c, **kw) for _ in range(c.num_hidden_layers)])
        self.norm_out = _AdaLNZero(D, 2, **kw)
        self.proj_out = nn.Linear(D, c.mel_dim, **kw)

    def _time_embed(self, t, dtype):
        half = 128
        f = torch.exp(-math.log(10000.0) * torch.arange(half, device=t.device) / (half - 1))
        a = (t.float() * 1000.0)[:, None] * f[None]
        return self.time_mlp(torch.cat([a.sin(), a.cos()], -1).to(dtype))

    def _band_mask(self, T, device):
        c = self.c
        blk = torch.arange(T, device=device) // c.block_size
        d = blk[None, :] - blk[:, None]
        return (d >= -c.look_backward_blocks) & (d <= c.look_ahead_blocks)

    def velocity(self, x, t, code_emb, spk, drop: bool):
        """x [B, T, mel]; code_emb [B, T, emb]; spk [B, speaker_dim]; drop: the null branch."""
        B, T, _ = x.shape
        if drop:
            code_emb, spk = torch.zeros_like(code_emb), torch.zeros_like(spk)
        h = self.in_proj(torch.cat([x, code_emb, spk[:, None].expand(B, T, -1)], -1))
        emb = self._time_embed(t.expand(B), x.dtype)
        Dh = self.c.head_dim
        inv = 1.0 / (10000 ** (torch.arange(0, Dh, 2, device=x.device).float() / Dh))
        ang = torch.arange(T, device=x.device).float()[:, None] * inv[None]
        cos, sin = ang.cos().to(x.dtype)[None, None], ang.sin().to(x.dtype)[None, None]
        mask = self._band_mask(T, x.device)
        for blk in self.blocks:
            h = blk(h, emb, cos, sin, mask)
        sh, sc = self.norm_out(emb)
        h = F.layer_norm(h, (h.shape[-1],)) * (1 + sc[:, None]) + sh[:, None]
        return self.proj_out(h)

    @torch.no_grad()
    def sample(self, codes, spk=None, num_steps=None, guidance_scale=None, sway=None, generator=None):
        """codes [B, T_code] -> mel [B, mel_dim, T_code * repeats]."""
        c = self.c
        B, Tc = codes.shape
        dev, dt = self.codec_embed.weight.device, self.codec_embed.weight.dtype
        emb = self.codec_embed(codes.clamp(0, c.num_embeds - 1)).repeat_interleave(c.repeats, dim=1)
        T = emb.shape[1]
        spk = torch.zeros(B, c.speaker_dim, device=dev, dtype=dt) if spk is None else spk.to(dev, dt)
        x0 = torch.randn(B, T, c.mel_dim, device=dev, dtype=torch.float32, generator=generator).to(dt)
        g = c.guidance_scale if guidance_scale is None else guidance_scale
        times = sway_time_grid(num_steps or c.num_steps, c.sway_coefficient if sway is None else sway, dev)

        def fn(t, x):
            v = self.velocity(x, t.reshape(1), emb, spk, drop=False)
            if g < 1e-5:
                return v
            return v + (v - self.velocity(x, t.reshape(1), emb, spk, drop=True)) * g

        mel = rk4_38_integrate(fn, x0, times)
        return mel.transpose(1, 2)


class SnakeBeta(nn.Module):
    """x + sin^2(alpha x) / beta with per-channel log-scale parameters."""

    def __init__(self, ch, **kw):
        super().__init__()
        self.alpha = nn.Parameter(torch.zeros(ch, **kw), requires_grad=False)
        self.beta = nn.Parameter(torch.zeros(ch, **kw), requires_grad=False)

    def forward(self, x):
        a, b = self.alpha.exp()[None, :, None], self.beta.exp()[None, :, None]
        return x + torch.sin(a * x) ** 2 / (b + 1e-9)


class AMPBlock(nn.Module):
    def __init__(self, ch, k, dilations, **kw):
        super().__init__()
        self.c1 = nn.ModuleList([nn.Conv1d(ch, ch, k, dilation=d, padding=(k - 1) * d // 2, **kw) for d in dilations])
        self.c2 = nn.ModuleList([nn.Conv1d(ch, ch, k, padding=(k - 1) // 2, **kw) for _ in dilations])
        self.a1 = nn.ModuleList([SnakeBeta(ch, **kw) for _ in dilations])
        self.a2 = nn.ModuleList([SnakeBeta(ch, **kw) for _ in dilations])

    def forward(self, x):
        for c1, c2, a1, a2 in zip(self.c1, self.c2, self.a1, self.a2):
            x = x + c2(a2(c1(a1(x))))
        return x


class BigVGAN(nn.Module):
    def __init__(self, c: BigVGANConfig, dtype, device):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.c = c
        ch = c.upsample_initial_channel
        self.conv_pre = nn.Conv1d(c.mel_dim, ch, 7, padding=3, **kw)
        self.ups, self.res = nn.ModuleList(), nn.ModuleList()
        for r, k in zip(c.upsample_rates, c.upsample_kernel_sizes):
            self.ups.append(nn.ConvTranspose1d(ch, ch // 2, k, stride=r, padding=(k - r) // 2, **kw))
            ch //= 2
            self.res.append(nn.ModuleList([AMPBlock(ch, rk, rd, **kw) for rk, rd in
                                           zip(c.resblock_kernel_sizes, c.resblock_dilation_sizes)]))
        self.act_post = SnakeBeta(ch, **kw)
        self.conv_post = nn.Conv1d(ch, 1, 7, padding=3, bias=False, **kw)

    @torch.no_grad()
    def forward(self, mel):
        """mel [B, mel_dim, T] -> waveform [B, T * total_upsample] in [-1, 1]."""
        x = self.conv_pre(mel)
        for up, blocks in zip(self.ups, self.res):
            x = up(x)
            x = sum(b(x) for b in blocks) / len(blocks)
        x = self.conv_post(self.act_post(x))
        return torch.clamp(x.float(), -1.0, 1.0)[:, 0]


class Qwen25OmniToken2Wav(StageModel):
    engine_output_type = "audio"
    is_generation_model = True

    def __init__(self, cfg: Qwen25OmniConfig, dtype=torch.bfloat16, device=None):
        super().__init__(None, dtype, device)
        self.cfg = cfg
        self.dit = Token2WavDiT(cfg.dit, dtype, device)
        self.vocoder = BigVGAN(cfg.bigvgan, dtype, device)
        self.voices: dict[str, torch.Tensor] = {}       # voice name -> conditioning vector

    def register_voice(self, name: str, vec: torch.Tensor) -> None:
        self.voices[name] = vec.reshape(1, -1)

    @torch.no_grad()
    def codes_to_wav(self, codes: torch.Tensor, voice: str | None = None, seed: int = 0, **kw) -> torch.Tensor:
        dev = self.dit.codec_embed.weight.device
        codes = codes.long().to(dev).reshape(1, -1) if codes.dim() <= 1 else codes.long().to(dev)
        if codes.shape[1] == 0:
            return torch.zeros(codes.shape[0], 0, device=dev)
        gen = torch.Generator(device=dev).manual_seed(int(seed))
        mel = self.dit.sample(codes, self.voices.get(voice or "default"), generator=gen, **kw)
        return self.vocoder(mel)

    def generate_for(self, req, start, n):
        info = req.additional_information
        codes = info.get("codes")
        if codes is None:
            codes = torch.tensor(req.prompt_token_ids[start:start + n], dtype=torch.long)
        codes = torch.as_tensor(codes).long().reshape(-1)
        wav = self.codes_to_wav(codes, voice=info.get("voice"), seed=req.sampling_params.seed or 0)
        return {"audio": wav[0].float(), "sample_rate": self.cfg.bigvgan.sample_rate}
