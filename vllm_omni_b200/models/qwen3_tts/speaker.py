"""Speaker encoder of Qwen3-TTS: 24 kHz reference audio -> log-mel spectrogram -> ECAPA-TDNN ->
one x-vector of the talker's width, which stands in the prompt where a named voice's codec token
would (vllm_omni/model_executor/models/qwen3_tts/modeling_qwen3_tts.py:59-430, 1917-1931).

The mel filterbank is the Slaney-scale, area-normalised triangular bank (linear below 1 kHz,
logarithmic above; each filter divided by half its bandwidth) that the reference takes from librosa;
it is computed here so that no audio library is needed.  The network is the same ECAPA-TDNN as
Qwen2.5-Omni's token2wav speaker encoder (parameter names ``blocks.N.*``, ``mfa``, ``asp``, ``fc``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from ..qwen2_5_omni.token2wav import ECAPA


@dataclass
class SpeakerEncoderConfig:
    mel_dim: int = 128
    enc_dim: int = 1024
    enc_channels: tuple = (512, 512, 512, 512, 1536)
    enc_kernel_sizes: tuple = (5, 3, 3, 3, 1)
    enc_dilations: tuple = (1, 2, 3, 4, 1)
    enc_attention_channels: int = 128
    enc_res2net_scale: int = 8
    enc_se_channels: int = 128
    sample_rate: int = 24000

    @classmethod
    def from_dict(cls, d: dict) -> "SpeakerEncoderConfig":
        keys = set(cls.__dataclass_fields__)
        return cls(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in d.items() if k in keys})


def _hz_to_mel(f: torch.Tensor) -> torch.Tensor:
    f_sp, min_log_hz = 200.0 / 3, 1000.0
    min_log_mel, logstep = min_log_hz / f_sp, math.log(6.4) / 27.0
    return torch.where(f >= min_log_hz, min_log_mel + torch.log(f.clamp(min=1e-10) / min_log_hz) / logstep, f / f_sp)


def _mel_to_hz(m: torch.Tensor) -> torch.Tensor:
    f_sp, min_log_hz = 200.0 / 3, 1000.0
    min_log_mel, logstep = min_log_hz / f_sp, math.log(6.4) / 27.0
    return torch.where(m >= min_log_mel, min_log_hz * torch.exp(logstep * (m - min_log_mel)), f_sp * m)


def mel_filterbank_slaney(sr: int, n_fft: int, n_mels: int, fmin: float = 0.0, fmax: float | None = None) -> torch.Tensor:
    """[n_mels, n_fft / 2 + 1] triangular filters, Slaney mel scale, each scaled by 2 / bandwidth."""
    fmax = sr / 2.0 if fmax is None else float(fmax)
    fft_f = torch.linspace(0, sr / 2.0, n_fft // 2 + 1, dtype=torch.float64)
    lo, hi = _hz_to_mel(torch.tensor(float(fmin), dtype=torch.float64)), _hz_to_mel(torch.tensor(fmax, dtype=torch.float64))
    edges = _mel_to_hz(torch.linspace(float(lo), float(hi), n_mels + 2, dtype=torch.float64))
    width = edges[1:] - edges[:-1]
    ramps = edges[:, None] - fft_f[None]
    lower = -ramps[:-2] / width[:-1, None]
    upper = ramps[2:] / width[1:, None]
    bank = torch.clamp(torch.minimum(lower, upper), min=0)
    bank = bank * (2.0 / (edges[2:] - edges[:-2]))[:, None]
    return bank.float()


def mel_spectrogram(wav: torch.Tensor, n_fft=1024, num_mels=128, sampling_rate=24000, hop_size=256, win_size=1024,
                    fmin=0, fmax=12000) -> torch.Tensor:
    """wav [B, T] in [-1, 1] -> log-mel [B, num_mels, frames]: reflect padding of (n_fft - hop) / 2
    on both sides, Hann window, magnitude sqrt(re^2 + im^2 + 1e-9), log(clamp(mel, 1e-5))."""
    bank = mel_filterbank_slaney(sampling_rate, n_fft, num_mels, fmin, fmax).to(wav.device)
    pad = (n_fft - hop_size) // 2
    y = F.pad(wav.float().unsqueeze(1), (pad, pad), mode="reflect").squeeze(1)
    spec = torch.stft(y, n_fft, hop_length=hop_size, win_length=win_size, window=torch.hann_window(win_size, device=wav.device),
                      center=False, normalized=False, onesided=True, return_complex=True)
    mag = torch.sqrt(torch.view_as_real(spec).pow(2).sum(-1) + 1e-9)
    return torch.log(torch.clamp(bank @ mag, min=1e-5))


def resample_sinc(wav: torch.Tensor, sr_in: int, sr_out: int) -> torch.Tensor:
    """Band-limited (windowed-sinc) resampling of [B, T] audio; used when the reference clip is not 24 kHz."""
    if sr_in == sr_out:
        return wav
    g = math.gcd(sr_in, sr_out)
    up, down = sr_out // g, sr_in // g
    cutoff = 0.5 / max(up, down)
    half = 16 * max(up, down)
    t = torch.arange(-half, half + 1, dtype=torch.float64)
    h = 2 * cutoff * torch.sinc(2 * cutoff * t) * torch.kaiser_window(2 * half + 1, periodic=False, beta=8.6, dtype=torch.float64)
    h = (h * up).float().to(wav.device)
    B, T = wav.shape
    x = torch.zeros(B, T * up, device=wav.device)
    x[:, ::up] = wav.float()
    y = F.conv1d(x[:, None], h[None, None], padding=half)[:, 0]
    return y[:, ::down].contiguous()


class Qwen3TTSSpeakerEncoder(ECAPA):
    """ECAPA-TDNN over the mel frames; kept in fp32 (a one-off per cloned voice)."""

    def __init__(self, cfg: SpeakerEncoderConfig, device=None):
        super().__init__(cfg)
        self.cfg = cfg
        self.to(device=device, dtype=torch.float32)
        for p in self.parameters():
            p.requires_grad_(False)

    @torch.no_grad()
    def embed_audio(self, wav: torch.Tensor, sr: int) -> torch.Tensor:
        """wav [T] or [1, T] -> x-vector [enc_dim]."""
        wav = wav.reshape(1, -1).to(next(self.parameters()).device)
        wav = resample_sinc(wav, int(sr), self.cfg.sample_rate)
        mel = mel_spectrogram(wav, num_mels=self.cfg.mel_dim, sampling_rate=self.cfg.sample_rate,
                              fmax=self.cfg.sample_rate // 2).transpose(1, 2)
        return self(mel)[0]

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        params = dict(self.named_parameters())
        loaded = set()
        for n, w in weights:
            if n in params:
                params[n].copy_(w.to(params[n].dtype))
                loaded.add(n)
        return loaded
