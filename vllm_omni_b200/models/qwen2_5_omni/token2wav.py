"""Qwen2.5-Omni token2wav ("code2wav" stage): codec tokens -> mel spectrogram by a flow-matching
DiT integrated with a Runge-Kutta (3/8 rule) solver under classifier-free guidance, then a
BigVGAN vocoder mel -> 24 kHz waveform
(vllm_omni/model_executor/models/qwen2_5_omni/qwen2_5_omni_token2wav.py:385-1860; module tree and
parameter names as in the Hugging Face checkpoint, ``token2wav.code2wav_dit_model.*`` and
``token2wav.code2wav_bigvgan_model.*``).

DiT input per mel frame: [noisy mel | speaker encoding of the reference mel (ECAPA-TDNN) | codec
embedding (each token repeated ``repeats`` times) | speaker x-vector], projected to the model width.
Blocks: AdaLN-zero from the time embedding, attention whose rotary embedding is applied to the FIRST
head only and which sees its own block of ``block_size`` frames plus, in selected layers, the
previous or the next block (this locality is what makes chunked streaming decode possible), GELU
MLP.  Sampling: x(0) ~ N(0, 1), time grid ``linspace(0, 1, num_steps)`` warped by
``t + s (cos(pi t / 2) - 1 + t)``, velocity ``v = v_cond + g (v_cond - v_null)`` with the null
branch dropping the reference mel, the x-vector and the codes.

BigVGAN: conv, then per up-sampling stage a transposed conv and the mean of three AMP residual
blocks whose SnakeBeta activations run at twice the rate between Kaiser-windowed-sinc up / down
filters (anti-aliasing), a last filtered activation and a conv to one channel.

The stage runs in fp32 like the reference (its checkpoint is fp32 and the solver is sensitive).
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


# ------------------------------------------------------------------------------ speaker encoder (ECAPA-TDNN)
class TDNNBlock(nn.Module):
    def __init__(self, cin, cout, k, dilation):
        super().__init__()
        self.conv = nn.Conv1d(cin, cout, k, dilation=dilation, padding="same", padding_mode="reflect")

    def forward(self, x):
        return F.relu(self.conv(x))


class Res2NetBlock(nn.Module):
    def __init__(self, ch, scale, k, dilation):
        super().__init__()
        self.scale = scale
        self.blocks = nn.ModuleList([TDNNBlock(ch // scale, ch // scale, k, dilation) for _ in range(scale - 1)])

    def forward(self, x):
        outs, y = [], None
        for i, part in enumerate(torch.chunk(x, self.scale, dim=1)):
            if i == 0:
                y = part
            elif i == 1:
                y = self.blocks[0](part)
            else:
                y = self.blocks[i - 1](part + y)
            outs.append(y)
        return torch.cat(outs, dim=1)


class SEBlock(nn.Module):
    def __init__(self, ch, se):
        super().__init__()
        self.conv1 = nn.Conv1d(ch, se, 1, padding="same", padding_mode="reflect")
        self.conv2 = nn.Conv1d(se, ch, 1, padding="same", padding_mode="reflect")

    def forward(self, x):
        s = torch.sigmoid(self.conv2(F.relu(self.conv1(x.mean(dim=2, keepdim=True)))))
        return x * s


class SERes2NetBlock(nn.Module):
    def __init__(self, cin, cout, scale, se, k, dilation):
        super().__init__()
        self.tdnn1 = TDNNBlock(cin, cout, 1, 1)
        self.res2net_block = Res2NetBlock(cout, scale, k, dilation)
        self.tdnn2 = TDNNBlock(cout, cout, 1, 1)
        self.se_block = SEBlock(cout, se)

    def forward(self, x):
        return self.se_block(self.tdnn2(self.res2net_block(self.tdnn1(x)))) + x


class AttentiveStatsPooling(nn.Module):
    def __init__(self, ch, att):
        super().__init__()
        self.tdnn = TDNNBlock(ch * 3, att, 1, 1)
        self.conv = nn.Conv1d(att, ch, 1, padding="same", padding_mode="reflect")

    @staticmethod
    def _stats(x, w):
        mean = (w * x).sum(2)
        std = torch.sqrt((w * (x - mean.unsqueeze(2)).pow(2)).sum(2).clamp(1e-12))
        return mean, std

    def forward(self, x):
        T = x.shape[-1]
        mean, std = self._stats(x, torch.full_like(x[:, :1], 1.0 / T))
        a = torch.cat([x, mean.unsqueeze(2).expand(-1, -1, T), std.unsqueeze(2).expand(-1, -1, T)], dim=1)
        a = F.softmax(self.conv(torch.tanh(self.tdnn(a))), dim=2)
        mean, std = self._stats(x, a)
        return torch.cat([mean, std], dim=1).unsqueeze(2)


class ECAPA(nn.Module):
    """Reference mel [B, T, mel] -> speaker encoding [B, enc_dim]."""

    def __init__(self, c: DiTConfig):
        super().__init__()
        ch, ks, ds = c.enc_channels, c.enc_kernel_sizes, c.enc_dilations
        self.blocks = nn.ModuleList([TDNNBlock(c.mel_dim, ch[0], ks[0], ds[0])])
        for i in range(1, len(ch) - 1):
            self.blocks.append(SERes2NetBlock(ch[i - 1], ch[i], c.enc_res2net_scale, c.enc_se_channels, ks[i], ds[i]))
        self.mfa = TDNNBlock(ch[-1], ch[-1], ks[-1], ds[-1])
        self.asp = AttentiveStatsPooling(ch[-1], c.enc_attention_channels)
        self.fc = nn.Conv1d(ch[-1] * 2, c.enc_dim, 1, padding="same", padding_mode="reflect")

    def forward(self, mel):
        x = mel.transpose(1, 2)
        feats = []
        for blk in self.blocks:
            x = blk(x)
            feats.append(x)
        x = self.mfa(torch.cat(feats[1:], dim=1))
        return self.fc(self.asp(x)).squeeze(-1)


# ------------------------------------------------------------------------------ DiT
class _ModLinear(nn.Module):
    """SiLU -> Linear(dim, n * dim): parameters ``linear.weight/bias``."""

    def __init__(self, dim, n):
        super().__init__()
        self.linear = nn.Linear(dim, n * dim)
        self.n = n

    def forward(self, emb):
        return self.linear(F.silu(emb)).chunk(self.n, dim=1)


class DiTAttention(nn.Module):
    def __init__(self, c: DiTConfig):
        super().__init__()
        D, inner = c.hidden_size, c.head_dim * c.num_attention_heads
        self.heads = c.num_attention_heads
        self.to_q, self.to_k, self.to_v = nn.Linear(D, inner), nn.Linear(D, inner), nn.Linear(D, inner)
        self.to_out = nn.ModuleList([nn.Linear(inner, D)])

    @staticmethod
    def _rot(x, cos, sin):
        """Pair-wise rotation of the FIRST head with the angle table tiled twice along the head width:
        element i of a pair (2j, 2j+1) uses angle index i mod (head_dim / 2)."""
        xr = torch.stack([-x[..., 1::2], x[..., 0::2]], dim=-1).flatten(-2)
        return x * cos + xr * sin

    def forward(self, x, cos, sin, mask):
        B, T, _ = x.shape
        q = self.to_q(x).view(B, T, self.heads, -1).transpose(1, 2)
        k = self.to_k(x).view(B, T, self.heads, -1).transpose(1, 2)
        v = self.to_v(x).view(B, T, self.heads, -1).transpose(1, 2)
        q = torch.cat([self._rot(q[:, :1], cos, sin), q[:, 1:]], dim=1)
        k = torch.cat([self._rot(k[:, :1], cos, sin), k[:, 1:]], dim=1)
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
        return self.to_out[0](o.transpose(1, 2).reshape(B, T, -1))


class DiTLayer(nn.Module):
    def __init__(self, c: DiTConfig, look_ahead: int, look_backward: int):
        super().__init__()
        D = c.hidden_size
        self.attn_norm = _ModLinear(D, 6)
        self.attn = DiTAttention(c)
        self.look_ahead, self.look_backward = look_ahead, look_backward
        inner = int(D * c.ff_mult)
        # indices 0 and 3 like the checkpoint's ModuleList [Linear, GELU, Dropout, Linear]
        self.ff = nn.Module()
        self.ff.ff = nn.ModuleList([nn.Linear(D, inner), nn.Identity(), nn.Identity(), nn.Linear(inner, D)])

    def forward(self, x, temb, cos, sin, block_diff):
        D = x.shape[-1]
        s1, c1, g1, s2, c2, g2 = self.attn_norm(temb)
        h = F.layer_norm(x, (D,), eps=1e-6) * (1 + c1[:, None]) + s1[:, None]
        mask = (block_diff >= -self.look_backward) & (block_diff <= self.look_ahead)
        x = x + g1[:, None] * self.attn(h, cos, sin, mask)
        h = F.layer_norm(x, (D,), eps=1e-6) * (1 + c2[:, None]) + s2[:, None]
        return x + g2[:, None] * self.ff.ff[3](F.gelu(self.ff.ff[0](h), approximate="tanh"))


class Token2WavDiT(nn.Module):
    def __init__(self, c: DiTConfig):
        super().__init__()
        self.c = c
        D = c.hidden_size
        self.time_embed = nn.Module()
        self.time_embed.time_mlp = nn.ModuleList([nn.Linear(256, D), nn.Identity(), nn.Linear(D, D)])
        self.text_embed = nn.Module()
        self.text_embed.codec_embed = nn.Embedding(c.num_embeds + 1, c.emb_dim)
        self.input_embed = nn.Module()
        self.input_embed.proj = nn.Linear(c.mel_dim + c.enc_dim + c.enc_emb_dim + c.emb_dim, D)
        self.input_embed.spk_encoder = ECAPA(c)
        self.transformer_blocks = nn.ModuleList([DiTLayer(c, int(i in c.look_ahead_layers), int(i in c.look_backward_layers))
                                                 for i in range(c.num_hidden_layers)])
        self.norm_out = _ModLinear(D, 2)
        self.proj_out = nn.Linear(D, c.mel_dim)

    def _time(self, t):
        half = 128
        f = torch.exp(torch.arange(half, device=t.device).float() * -(math.log(10000) / (half - 1)))
        a = 1000.0 * t.float()[:, None] * f[None]
        h = torch.cat([a.sin(), a.cos()], dim=-1).to(t.dtype)
        m = self.time_embed.time_mlp
        return m[2](F.silu(m[0](h)))

    def block_diff(self, T, device):
        blk = torch.arange(T, device=device) // self.c.block_size
        return blk[None, :] - blk[:, None]

    def forward(self, x, ref_mel, xvec, codes, t, apply_cfg=True):
        """x [B, T, mel] noisy mel, ref_mel [B, T_ref, mel], xvec [B, T, enc_emb_dim] (already repeated
        over time), codes [B, T / repeats], t scalar or [B].  With ``apply_cfg`` the batch is doubled:
        rows [0, B) conditional, rows [B, 2B) with reference, x-vector and codes dropped."""
        c = self.c
        B = x.shape[0]
        t = t.reshape(-1).expand(B) if t.numel() == 1 else t
        temb = self._time(t.to(x.dtype))
        emb = self.text_embed.codec_embed
        code = emb(codes).repeat_interleave(c.repeats, dim=1)
        if apply_cfg:
            null = emb(torch.zeros_like(codes)).repeat_interleave(c.repeats, dim=1)
            x, xvec = torch.cat([x, x]), torch.cat([xvec, torch.zeros_like(xvec)])
            ref_mel, code = torch.cat([ref_mel, torch.zeros_like(ref_mel)]), torch.cat([code, null])
            temb = torch.cat([temb, temb])
        T = x.shape[1]
        spk = self.input_embed.spk_encoder(ref_mel).unsqueeze(1).expand(-1, T, -1)
        h = self.input_embed.proj(torch.cat([x, spk, code, xvec], dim=-1))
        inv = 1.0 / (c.rope_theta ** (torch.arange(0, c.head_dim, 2, device=x.device).float() / c.head_dim))
        ang = torch.arange(T, device=x.device).float()[:, None] * inv[None]
        ang = torch.cat([ang, ang], dim=-1)
        cos, sin = ang.cos().to(x.dtype)[None, None], ang.sin().to(x.dtype)[None, None]
        diff = self.block_diff(T, x.device)
        for blk in self.transformer_blocks:
            h = blk(h, temb, cos, sin, diff)
        scale, shift = self.norm_out(temb)
        h = F.layer_norm(h, (h.shape[-1],), eps=1e-6) * (1 + scale)[:, None] + shift[:, None]
        return self.proj_out(h)

    @torch.no_grad()
    def sample(self, codes, xvec=None, ref_mel=None, num_steps=None, guidance_scale=None, sway=None, generator=None,
               noise=None, solver="rk4"):
        """codes [B, T_code] -> mel [B, mel_dim, T_code * repeats].  ``solver``: "rk4" (3/8 rule, the
        Qwen2.5-Omni vocoder) or "euler" (one evaluation per interval, the Qwen3-TTS 25 Hz decoder)."""
        c = self.c
        B, Tc = codes.shape
        p = self.proj_out.weight
        dev, dt = p.device, p.dtype
        T = Tc * c.repeats
        xvec = torch.zeros(B, c.enc_emb_dim, device=dev, dtype=dt) if xvec is None else xvec.to(dev, dt).reshape(B, -1)
        ref_mel = torch.zeros(B, max(8, c.enc_kernel_sizes[0]), c.mel_dim, device=dev, dtype=dt) if ref_mel is None \
            else ref_mel.to(dev, dt)
        xv = xvec.unsqueeze(1).expand(-1, T, -1)
        x0 = noise.to(dev, dt) if noise is not None else \
            torch.randn(B, T, c.mel_dim, device=dev, dtype=torch.float32, generator=generator).to(dt)
        g = c.guidance_scale if guidance_scale is None else guidance_scale
        times = sway_time_grid(num_steps or c.num_steps, c.sway_coefficient if sway is None else sway, dev).to(dt)

        def fn(t, x):
            if g < 1e-5:
                return self(x, ref_mel, xv, codes, t, apply_cfg=False)
            cond, null = self(x, ref_mel, xv, codes, t, apply_cfg=True).chunk(2, dim=0)
            return cond + (cond - null) * g

        if solver == "euler":
            x = x0
            for t0, t1 in zip(times[:-1], times[1:]):
                x = x + fn(t0, x) * (t1 - t0)
            return x.transpose(1, 2)
        return rk4_38_integrate(fn, x0, times).transpose(1, 2)


# ------------------------------------------------------------------------------ BigVGAN
def kaiser_sinc_filter(cutoff: float, half_width: float, k: int) -> torch.Tensor:
    half = k // 2
    att = 2.285 * (half - 1) * math.pi * 4 * half_width + 7.95
    beta = 0.1102 * (att - 8.7) if att > 50 else (0.5842 * (att - 21) ** 0.4 + 0.07886 * (att - 21) if att >= 21 else 0.0)
    win = torch.kaiser_window(k, beta=beta, periodic=False, dtype=torch.float32)
    t = (torch.arange(-half, half) + 0.5) if k % 2 == 0 else (torch.arange(k) - half)
    f = 2 * cutoff * win * torch.sinc(2 * cutoff * t)
    return (f / f.sum()).view(1, 1, k)


class SnakeBeta(nn.Module):
    """x + sin^2(x e^alpha) / e^beta, per channel."""

    def __init__(self, ch):
        super().__init__()
        self.alpha = nn.Parameter(torch.zeros(ch), requires_grad=False)
        self.beta = nn.Parameter(torch.zeros(ch), requires_grad=False)

    def forward(self, x):
        a, b = self.alpha.exp()[None, :, None], self.beta.exp()[None, :, None]
        return x + torch.sin(x * a).pow(2) / (b + 1e-9)


class FilteredActivation(nn.Module):
    """2x up-sample (windowed sinc), activation, 2x down-sample: the activation's harmonics above the
    original Nyquist frequency are removed again.  Parameters: ``act.alpha / act.beta``."""

    def __init__(self, ch, k=12):
        super().__init__()
        self.act = SnakeBeta(ch)
        self.k = k
        self.register_buffer("up_filter", kaiser_sinc_filter(0.25, 0.3, k), persistent=False)
        self.register_buffer("down_filter", kaiser_sinc_filter(0.25, 0.3, k), persistent=False)

    def forward(self, x):
        C, k = x.shape[1], self.k
        pad = k // 2 - 1
        y = F.pad(x, (pad, pad), mode="replicate")
        y = 2 * F.conv_transpose1d(y, self.up_filter.expand(C, -1, -1), stride=2, groups=C)
        pl, pr = pad * 2 + (k - 2) // 2, pad * 2 + (k - 2 + 1) // 2
        y = self.act(y[..., pl:-pr])
        y = F.pad(y, (k // 2 - (1 - k % 2), k // 2), mode="replicate")
        return F.conv1d(y, self.down_filter.expand(C, -1, -1), stride=2, groups=C)


class AMPBlock(nn.Module):
    def __init__(self, ch, k, dilations):
        super().__init__()
        pad = lambda d: int((k * d - d) / 2)
        self.convs1 = nn.ModuleList([nn.Conv1d(ch, ch, k, dilation=d, padding=pad(d)) for d in dilations])
        self.convs2 = nn.ModuleList([nn.Conv1d(ch, ch, k, padding=pad(1)) for _ in dilations])
        self.activations = nn.ModuleList([FilteredActivation(ch) for _ in range(2 * len(dilations))])

    def forward(self, x):
        for i, (c1, c2) in enumerate(zip(self.convs1, self.convs2)):
            x = x + c2(self.activations[2 * i + 1](c1(self.activations[2 * i](x))))
        return x


class BigVGAN(nn.Module):
    def __init__(self, c: BigVGANConfig):
        super().__init__()
        self.c = c
        ch = c.upsample_initial_channel
        self.conv_pre = nn.Conv1d(c.mel_dim, ch, 7, padding=3)
        self.ups = nn.ModuleList([nn.ModuleList([nn.ConvTranspose1d(ch // 2 ** i, ch // 2 ** (i + 1), k, r, padding=(k - r) // 2)])
                                  for i, (r, k) in enumerate(zip(c.upsample_rates, c.upsample_kernel_sizes))])
        self.resblocks = nn.ModuleList([AMPBlock(ch // 2 ** (i + 1), k, d) for i in range(len(c.upsample_rates))
                                        for k, d in zip(c.resblock_kernel_sizes, c.resblock_dilation_sizes)])
        last = ch // 2 ** len(c.upsample_rates)
        self.activation_post = FilteredActivation(last)
        self.conv_post = nn.Conv1d(last, 1, 7, padding=3, bias=False)

    @staticmethod
    def process_mel(mel):
        """log-mel -> dB (floor -115 dB, -20 dB reference) -> [-1, 1]."""
        amp = torch.exp(mel)
        floor = math.exp(-115 / 20.0 * math.log(10))
        db = 20 * torch.log10(amp.clamp(min=floor)) - 20
        return torch.clamp(2 * ((db + 115) / 115) - 1, -1, 1)

    # ------------------------------------------------------------------ channels-last path (own kernels)
    def _packed(self, m, dtype):
        """Weights of a convolution in the layout of the 1-D implicit GEMM, packed once per module."""
        from ...ops import conv as CV
        cache = self.__dict__.setdefault("_pk", {})
        key = (id(m), m.weight._version, dtype)
        if key not in cache:
            b = m.bias.data if m.bias is not None else None
            if isinstance(m, nn.ConvTranspose1d):
                cache[key] = CV.pack_conv_transpose1d_weight(m.weight.data, b, m.stride[0], m.padding[0], dtype)
            else:
                cache[key] = CV.pack_conv1d_weight(m.weight.data, b, dtype)
        return cache[key]

    def _conv_nlc(self, m, x, residual=None):
        from ...ops import conv as CV
        k, d = m.kernel_size[0], m.dilation[0]
        pw, pb = self._packed(m, x.dtype)
        y = CV.conv1d_nlc(x, pw, pb, k, m.in_channels, d, m.padding[0], residual=residual)
        return y if y.shape[-1] == m.out_channels else y[..., :m.out_channels]

    def _act_nlc(self, fa, x):
        from ...ops import conv as CV
        cache = self.__dict__.setdefault("_ab", {})
        key = (id(fa), fa.act.alpha._version, fa.act.beta._version)
        if key not in cache:
            cache[key] = (fa.act.alpha.float().exp().contiguous(), (1.0 / (fa.act.beta.float().exp() + 1e-9)).contiguous(),
                          fa.up_filter.float().flatten().contiguous(), fa.down_filter.float().flatten().contiguous())
        a, ib, fu, fd = cache[key]
        return CV.aa_snake_nlc(x.contiguous(), a, ib, fu, fd)

    @torch.no_grad()
    def forward_nlc(self, mel):
        """Same network on [B, T, C] tensors: the convolutions are the 1-D implicit GEMM (transposed ones as one
        stride-1 convolution on phase-stacked weights), every anti-aliased activation is one fused kernel, the
        residual adds ride in the GEMM epilogues (ops/conv.py)."""
        from ...ops import conv as CV
        n = len(self.c.resblock_kernel_sizes)
        dt = self.conv_pre.weight.dtype
        x = self.process_mel(mel).transpose(1, 2).to(dt)
        pad_c = (-x.shape[-1]) % 8
        if pad_c:                                          # TMA rows start on 16 bytes
            x = F.pad(x, (0, pad_c))
        x = self._conv_nlc(self.conv_pre, x.contiguous())
        for i, up in enumerate(self.ups):
            m = up[0]
            k, r, p = m.kernel_size[0], m.stride[0], m.padding[0]
            t_out = (x.shape[1] - 1) * r - 2 * p + k
            y = CV.conv_transpose1d_nlc(x, self._packed(m, x.dtype), m.in_channels, r, t_out)
            x = (y if y.shape[-1] == m.out_channels else y[..., :m.out_channels]).contiguous()
            acc = None
            for j in range(n):
                blk = self.resblocks[i * n + j]
                h = x
                for q, (c1, c2) in enumerate(zip(blk.convs1, blk.convs2)):
                    t = self._conv_nlc(c1, self._act_nlc(blk.activations[2 * q], h))
                    h = self._conv_nlc(c2, self._act_nlc(blk.activations[2 * q + 1], t), residual=h)
                acc = h.float() if acc is None else acc + h.float()
            x = (acc / n).to(dt)
        x = self._conv_nlc(self.conv_post, self._act_nlc(self.activation_post, x))
        return torch.clamp(x[..., 0].float(), -1.0, 1.0)

    def use_nlc(self, mel) -> bool:
        forced = getattr(self, "vocoder_layout", None)
        if forced is not None:
            return forced == "nlc"
        import os
        return (mel.is_cuda and self.conv_pre.weight.dtype == torch.bfloat16 and os.environ.get("OMNI_VOCODER_NLC", "1") != "0"
                and all(ch % 8 == 0 for ch in (self.conv_pre.out_channels, self.conv_post.in_channels)))

    @torch.no_grad()
    def forward(self, mel):
        """mel [B, mel_dim, T] -> waveform [B, T * total_upsample] in [-1, 1]."""
        if self.use_nlc(mel):
            return self.forward_nlc(mel)
        n = len(self.c.resblock_kernel_sizes)
        x = self.conv_pre(self.process_mel(mel))
        for i, up in enumerate(self.ups):
            x = up[0](x)
            x = sum(self.resblocks[i * n + j](x) for j in range(n)) / n
        x = self.conv_post(self.activation_post(x))
        return torch.clamp(x.float(), -1.0, 1.0)[:, 0]


# ------------------------------------------------------------------------------ stage
class Qwen25OmniToken2Wav(StageModel):
    engine_output_type = "audio"
    is_generation_model = True

    def __init__(self, cfg: Qwen25OmniConfig, dtype=torch.float32, device=None):
        super().__init__(None, torch.float32, device)
        self.cfg = cfg
        self.code2wav_dit_model = Token2WavDiT(cfg.dit).to(device=device, dtype=torch.float32)
        self.code2wav_bigvgan_model = BigVGAN(cfg.bigvgan).to(device=device, dtype=torch.float32)
        for p in self.parameters():
            p.requires_grad_(False)
        self.voices: dict[str, tuple] = {}       # voice name -> (x-vector [enc_emb_dim], reference mel [T_ref, mel_dim])

    @property
    def dit(self):
        return self.code2wav_dit_model

    @property
    def vocoder(self):
        return self.code2wav_bigvgan_model

    def register_voice(self, name: str, xvec: torch.Tensor, ref_mel: torch.Tensor | None = None) -> None:
        self.voices[name] = (xvec.reshape(1, -1), None if ref_mel is None else ref_mel.reshape(1, -1, self.cfg.dit.mel_dim))

    @torch.no_grad()
    def codes_to_wav(self, codes: torch.Tensor, voice: str | None = None, seed: int = 0, **kw) -> torch.Tensor:
        dev = self.dit.proj_out.weight.device
        codes = codes.long().to(dev).reshape(1, -1) if codes.dim() <= 1 else codes.long().to(dev)
        if codes.shape[1] == 0:
            return torch.zeros(codes.shape[0], 0, device=dev)
        codes = codes.clamp(0, self.cfg.dit.num_embeds)
        gen = torch.Generator(device=dev).manual_seed(int(seed))
        xvec, ref = self.voices.get(voice or "default", (None, None))
        mel = self.dit.sample(codes, xvec, ref, generator=gen, **kw)
        return self.vocoder(mel)

    def generate_for(self, req, start, n):
        info = req.additional_information
        codes = info.get("codes")
        if codes is None:
            codes = torch.tensor(req.prompt_token_ids[start:start + n], dtype=torch.long)
        codes = torch.as_tensor(codes).long().reshape(-1)
        wav = self.codes_to_wav(codes, voice=info.get("voice"), seed=req.sampling_params.seed or 0)
        return {"audio": wav[0].float(), "sample_rate": self.cfg.bigvgan.sample_rate}

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        """Checkpoint names under ``token2wav.``; other stages' tensors are ignored."""
        own = dict(self.named_parameters())
        loaded = set()
        for full, w in weights:
            if full.startswith(("thinker.", "talker.")):
                continue
            n = full[len("token2wav."):] if full.startswith("token2wav.") else full
            n = n.replace(".attn_norm.linear.", ".attn_norm.linear.")          # same tree; kept for clarity
            if n in own:
                own[n].copy_(w.to(own[n].dtype).reshape(own[n].shape))
                loaded.add(full)
        return loaded
