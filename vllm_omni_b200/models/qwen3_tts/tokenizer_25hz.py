"""Qwen3-TTS 25 Hz speech tokenizer (``model_type = qwen3_tts_tokenizer_25hz``): a Whisper-style
encoder whose sixth block's output is vector-quantised into ONE codebook stream at 25 codes per
second of 16 kHz audio (640 samples: two encoder positions of two mel frames each), and a decoder that is a
block-causal flow-matching transformer over mel frames followed by a BigVGAN vocoder
(vllm_omni/model_executor/models/qwen3_tts/tokenizer_25hz/modeling_qwen3_tts_tokenizer_v1.py:1234-1345
``Qwen3TTSTokenizerV1Decoder`` / ``...Encoder``, :1365-1523 ``Qwen3TTSTokenizerV1Model.encode/decode``,
vq/whisper_encoder.py, vq/speech_vq.py:178-403 ``WhisperEncoderVQ``, vq/core_vq.py:185-212).

The decoder's two networks are the ones the Qwen2.5-Omni vocoder stage already runs here
(``Token2WavDiT`` and ``BigVGAN``, the latter on the channels-last conv kernels on a GPU); this
decoder integrates the flow with plain Euler steps instead of the 3/8 rule.  The encoder is a
one-off per cloned voice and stays in fp32 PyTorch: only the blocks up to the quantiser are built.

Checkpoint names: ``encoder.tokenizer.{conv1,conv2,blocks.N.{attn_ln,attn.{query,key,value,out},
mlp_ln,mlp.0,mlp.2},audio_vq_downsample,audio_quantizer.rvqs.0.embed,
audio_quantizer.rvqs.0.layers.0.project_in}``, ``decoder.dit.*``, ``decoder.bigvgan.*``.

The reference obtains the speaker x-vector from an ONNX network through onnxruntime and normalises
the clip with sox; neither library exists here, so the x-vector comes from a callable the caller
registers (``set_xvector_extractor``) and the level normalisation (peak at -6 dB) is done inline.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F
from torch import nn

from ..qwen2_5_omni.config import BigVGANConfig, DiTConfig
from ..qwen2_5_omni.token2wav import BigVGAN, Token2WavDiT
from .speaker import mel_filterbank_slaney, mel_spectrogram

WHISPER_N_FFT = 400
WHISPER_HOP = 160


@dataclass
class Tokenizer25HzEncoderConfig:
    n_mels: int = 128
    n_ctx: int = 1500
    n_state: int = 1280
    n_head: int = 20
    n_layer: int = 32
    n_window: int = 100                     # attention window, in positions after the stride-2 conv
    audio_vq_layers: int = 6                # the quantiser sits after this many blocks
    audio_vq_codebook_size: int = 32768
    audio_vq_codebook_dim: int | None = 1280
    audio_vq_ds_rate: int = 2               # encoder positions per code

    @classmethod
    def from_dict(cls, d: dict | None) -> "Tokenizer25HzEncoderConfig":
        d = d or {}
        return cls(**{k: d[k] for k in cls.__dataclass_fields__ if k in d})


@dataclass
class Tokenizer25HzConfig:
    encoder: Tokenizer25HzEncoderConfig = field(default_factory=Tokenizer25HzEncoderConfig)
    dit: DiTConfig = field(default_factory=DiTConfig)
    bigvgan: BigVGANConfig = field(default_factory=BigVGANConfig)
    input_sample_rate: int = 24000
    output_sample_rate: int = 24000
    decode_upsample_rate: int = 1920        # output samples per code
    encode_downsample_rate: int = 1920

    @classmethod
    def from_dict(cls, d: dict | None) -> "Tokenizer25HzConfig":
        d = d or {}
        dec = d.get("decoder_config") or {}
        top = {k: d[k] for k in ("input_sample_rate", "output_sample_rate", "decode_upsample_rate",
                                 "encode_downsample_rate") if k in d}
        return cls(encoder=Tokenizer25HzEncoderConfig.from_dict(d.get("encoder_config")),
                   dit=DiTConfig.from_dict(dec.get("dit_config") or {}),
                   bigvgan=BigVGANConfig.from_dict(dec.get("bigvgan_config") or {}), **top)

    @classmethod
    def tiny(cls) -> "Tokenizer25HzConfig":
        enc = Tokenizer25HzEncoderConfig(n_mels=16, n_ctx=64, n_state=32, n_head=2, n_layer=3, n_window=8,
                                         audio_vq_layers=2, audio_vq_codebook_size=64, audio_vq_codebook_dim=32)
        dit = DiTConfig(hidden_size=32, num_hidden_layers=2, num_attention_heads=2, head_dim=16, mel_dim=8, num_embeds=65,
                        emb_dim=16, block_size=4, look_ahead_layers=(1,), look_backward_layers=(0,), enc_emb_dim=8,
                        enc_dim=8, enc_channels=(8, 8, 8, 8, 24), enc_attention_channels=4, enc_se_channels=4, num_steps=3)
        voc = BigVGANConfig(mel_dim=8, upsample_initial_channel=16, upsample_rates=(2, 2), upsample_kernel_sizes=(4, 4),
                            resblock_kernel_sizes=(3,), resblock_dilation_sizes=((1, 3),))
        return cls(encoder=enc, dit=dit, bigvgan=voc, decode_upsample_rate=2 * 4)


def whisper_log_mel(audio: torch.Tensor, n_mels: int, padding: int = 0) -> torch.Tensor:
    """[T] samples at 16 kHz framing -> [n_mels, frames] Whisper features: 400-point Hann STFT every 160
    samples (centred), the last frame dropped, power through a Slaney filterbank, log10 floored at 1e-10
    and at 8 below the clip's maximum, then (x + 4) / 4."""
    audio = audio.float()
    if padding > 0:
        audio = F.pad(audio, (0, padding))
    win = torch.hann_window(WHISPER_N_FFT, device=audio.device)
    spec = torch.stft(audio, WHISPER_N_FFT, WHISPER_HOP, window=win, return_complex=True)
    power = spec[..., :-1].abs() ** 2
    bank = mel_filterbank_slaney(16000, WHISPER_N_FFT, n_mels).to(audio.device)
    x = torch.clamp(bank @ power, min=1e-10).log10()
    x = torch.maximum(x, x.max() - 8.0)
    return (x + 4.0) / 4.0


def frames_after_cnn(t: int) -> int:
    """Positions left of ``t`` mel frames by the k3 s1 p1 conv and the k3 s2 p1 conv."""
    return (t + 2 - 3) // 2 + 1


def sinusoid_table(length: int, channels: int, max_timescale: float = 10000.0) -> torch.Tensor:
    inc = math.log(max_timescale) / (channels // 2 - 1)
    inv = torch.exp(-inc * torch.arange(channels // 2))
    ang = torch.arange(length)[:, None] * inv[None]
    return torch.cat([ang.sin(), ang.cos()], dim=1)


class _Attn(nn.Module):
    def __init__(self, D: int, H: int):
        super().__init__()
        self.n_head = H
        self.query, self.key = nn.Linear(D, D), nn.Linear(D, D, bias=False)
        self.value, self.out = nn.Linear(D, D), nn.Linear(D, D)

    def forward(self, x: torch.Tensor, lens: list[int]) -> torch.Tensor:
        """x [sum(lens), D]: full attention inside each run of ``lens`` positions, none across runs."""
        N, D = x.shape
        H = self.n_head
        q, k, v = self.query(x), self.key(x), self.value(x)
        W = max(lens)
        if all(n == W for n in lens):
            shp = (len(lens), W, H, D // H)
            o = F.scaled_dot_product_attention(q.view(shp).transpose(1, 2), k.view(shp).transpose(1, 2),
                                               v.view(shp).transpose(1, 2))
            return self.out(o.transpose(1, 2).reshape(N, D))
        # ragged tails: pad every run to W and mask the padded keys
        idx = torch.zeros(len(lens), W, dtype=torch.long, device=x.device)
        keep = torch.zeros(len(lens), W, dtype=torch.bool, device=x.device)
        s = 0
        for i, n in enumerate(lens):
            idx[i, :n] = torch.arange(s, s + n, device=x.device)
            keep[i, :n] = True
            s += n
        g = lambda t: t[idx].view(len(lens), W, H, D // H).transpose(1, 2)
        o = F.scaled_dot_product_attention(g(q), g(k), g(v), attn_mask=keep[:, None, None, :])
        return self.out(o.transpose(1, 2).reshape(len(lens), W, D)[keep])


class _Block(nn.Module):
    def __init__(self, D: int, H: int):
        super().__init__()
        self.attn_ln, self.mlp_ln = nn.LayerNorm(D), nn.LayerNorm(D)
        self.attn = _Attn(D, H)
        self.mlp = nn.Sequential(nn.Linear(D, 4 * D), nn.GELU(), nn.Linear(4 * D, D))

    def forward(self, x, lens):
        x = x + self.attn(self.attn_ln(x), lens)
        return x + self.mlp(self.mlp_ln(x))


class Tokenizer25HzEncoder(nn.Module):
    """Mel -> codes.  Only the blocks in front of the quantiser exist: the later blocks, the pooling and the
    projection of the full audio encoder never run on the way to the code indices."""

    def __init__(self, c: Tokenizer25HzEncoderConfig, device=None):
        super().__init__()
        self.c = c
        D = c.n_state
        self.conv1 = nn.Conv1d(c.n_mels, D, 3, padding=1)
        self.conv2 = nn.Conv1d(D, D, 3, stride=2, padding=1)
        self.register_buffer("positional_embedding", sinusoid_table(c.n_ctx, D), persistent=False)
        self.blocks = nn.ModuleList([_Block(D, c.n_head) for _ in range(min(c.audio_vq_layers, c.n_layer))])
        r = c.audio_vq_ds_rate
        self.audio_vq_downsample = nn.Conv1d(D, D, r, stride=r) if r != 1 else nn.Identity()
        cd = c.audio_vq_codebook_dim or D
        self.project_in = nn.Linear(D, cd) if cd != D else nn.Identity()
        self.register_buffer("codebook", torch.zeros(c.audio_vq_codebook_size, cd))
        self.to(device=device, dtype=torch.float32)
        for p in self.parameters():
            p.requires_grad_(False)

    def speech_to_mel(self, wav: torch.Tensor) -> torch.Tensor:
        """The clip is zero-padded to a whole number of codes (160 * 2 * ds_rate samples each)."""
        step = WHISPER_HOP * 2 * self.c.audio_vq_ds_rate
        pad = math.ceil(wav.numel() / step) * step - wav.numel()
        return whisper_log_mel(wav.reshape(-1).to(self.conv1.weight.device), self.c.n_mels, pad)

    @torch.no_grad()
    def mel_to_codes(self, mels: list[torch.Tensor]) -> list[torch.Tensor]:
        c = self.c
        xs, lens, per_clip = [], [], []
        for mel in mels:
            n_clip = 0
            for part in mel.float().split(c.n_window * 2, dim=1):
                h = F.gelu(self.conv2(F.gelu(self.conv1(part[None]))))[0].transpose(0, 1)
                xs.append(h + self.positional_embedding[: h.shape[0]])
                lens.append(h.shape[0])
                n_clip += h.shape[0]
            per_clip.append(n_clip)
        x = torch.cat(xs, dim=0)
        for blk in self.blocks:
            x = blk(x, lens)
        # The down-sampling conv runs over the concatenation of all clips, as the reference does: every
        # clip holds a whole number of codes, so no window straddles two clips.
        x = self.audio_vq_downsample(x.transpose(0, 1)[None])[0].transpose(0, 1)
        x = self.project_in(x)
        e = self.codebook
        d = x.pow(2).sum(1, keepdim=True) - 2 * x @ e.t() + e.pow(2).sum(1)[None]
        codes = d.argmin(dim=-1)
        return list(codes.split([n // c.audio_vq_ds_rate for n in per_clip]))

    def quantize_speech(self, wavs: list[torch.Tensor]) -> list[torch.Tensor]:
        return self.mel_to_codes([self.speech_to_mel(w) for w in wavs])

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        own = dict(self.named_parameters())
        loaded = set()
        for name, w in weights:
            n = name[len("tokenizer."):] if name.startswith("tokenizer.") else name
            if n == "audio_quantizer.rvqs.0.embed":
                self.codebook.copy_(w.reshape(self.codebook.shape))
            elif n.startswith("audio_quantizer.rvqs.0.layers.0.project_in."):
                getattr(self.project_in, n.rsplit(".", 1)[1]).copy_(w)
            elif n in own:
                own[n].copy_(w.to(own[n].dtype).reshape(own[n].shape))
            else:
                continue
            loaded.add(name)
        return loaded


def peak_normalize(wav: torch.Tensor, db_level: float = -6.0) -> torch.Tensor:
    """Scale the clip so that its largest sample sits at ``db_level`` dBFS (what ``sox norm -6`` does)."""
    peak = wav.abs().max().clamp(min=1e-9)
    return wav * (10.0 ** (db_level / 20.0) / peak)


def reference_mel_16k(wav: torch.Tensor) -> torch.Tensor:
    """[T] at 16 kHz -> [frames, 80]: 1024-point STFT, hop 160, 640-sample Hann window, 0-8 kHz Slaney
    bank, log(clamp(., 1e-5)) (vq/speech_vq.py:27-128 ``MelSpectrogramFeatures``)."""
    m = mel_spectrogram(wav.reshape(1, -1), n_fft=1024, num_mels=80, sampling_rate=16000, hop_size=160, win_size=640,
                        fmin=0, fmax=8000)
    return m[0].transpose(0, 1)


class Qwen3TTSTokenizer25Hz(nn.Module):
    """``encode`` (clips -> codes, x-vectors, reference mels) and ``decode`` (those three -> waveforms)."""

    def __init__(self, cfg: Tokenizer25HzConfig | None = None, device=None, with_encoder: bool = True):
        super().__init__()
        self.cfg = cfg or Tokenizer25HzConfig()
        self.encoder = Tokenizer25HzEncoder(self.cfg.encoder, device) if with_encoder else None
        self.dit = Token2WavDiT(self.cfg.dit).to(device=device, dtype=torch.float32)
        self.bigvgan = BigVGAN(self.cfg.bigvgan).to(device=device, dtype=torch.float32)
        for p in self.parameters():
            p.requires_grad_(False)
        self._xvector_fn = None

    def set_xvector_extractor(self, fn) -> None:
        """``fn(wav_16k [T] float tensor) -> [enc_emb_dim]`` speaker embedding (unit norm is applied here)."""
        self._xvector_fn = fn

    @property
    def device(self):
        return self.dit.proj_out.weight.device

    @torch.no_grad()
    def encode(self, wavs: list[torch.Tensor], sr: int = 16000):
        """Clips -> (codes [T_i] each, x-vectors [enc_emb_dim] each, reference mels [frames_i, 80] each).
        The encoder's features are framed for 16 kHz audio; other rates are resampled first."""
        if self.encoder is None:
            raise RuntimeError("this tokenizer was built without its encoder")
        from .speaker import resample_sinc
        dev = self.device
        clips = [resample_sinc(w.reshape(1, -1).float().to(dev), sr, 16000)[0] for w in wavs]
        codes = self.encoder.quantize_speech(clips)
        xvecs, mels = [], []
        for w in clips:
            n = peak_normalize(w)
            if self._xvector_fn is not None:
                xv = F.normalize(torch.as_tensor(self._xvector_fn(n)).float().reshape(-1).to(dev), dim=0)
            else:
                xv = torch.zeros(self.cfg.dit.enc_emb_dim, device=dev)
            xvecs.append(xv)
            mels.append(reference_mel_16k(n))
        return codes, xvecs, mels

    @torch.no_grad()
    def decode(self, codes: torch.Tensor, xvectors: torch.Tensor, ref_mels: torch.Tensor, seed: int | None = 0,
               num_steps: int = 10, guidance_scale: float = 0.5, sway: float | None = -1.0, noise=None) -> list[torch.Tensor]:
        """codes [B, T] (0 pads a shorter row), xvectors [B, enc_emb_dim], ref_mels [B, frames, mel] ->
        one waveform per row, cut to (codes > 0).sum() * decode_upsample_rate samples."""
        dev = self.device
        codes = codes.long().to(dev)
        codes = codes[None] if codes.dim() == 1 else codes
        gen = None if seed is None else torch.Generator(device=dev).manual_seed(int(seed))
        mel = self.dit.sample(codes.clamp(0, self.cfg.dit.num_embeds), xvectors, ref_mels, num_steps=num_steps,
                              guidance_scale=guidance_scale, sway=sway, generator=gen, noise=noise, solver="euler")
        wav = self.bigvgan(mel)
        wav = wav.reshape(codes.shape[0], -1)
        keep = (codes > 0).sum(1) * self.cfg.decode_upsample_rate
        return [w[: int(n)] for w, n in zip(wav, keep)]

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        dit, voc = dict(self.dit.named_parameters()), dict(self.bigvgan.named_parameters())
        loaded, enc = set(), []
        for name, w in weights:
            if name.startswith("encoder."):
                enc.append((name, w))
                continue
            for pre, own in (("decoder.dit.", dit), ("decoder.bigvgan.", voc)):
                n = name[len(pre):]
                if name.startswith(pre) and n in own:
                    own[n].copy_(w.to(own[n].dtype).reshape(own[n].shape))
                    loaded.add(name)
        if self.encoder is not None and enc:
            got = self.encoder.load_weights((n[len("encoder."):], w) for n, w in enc)
            loaded |= {"encoder." + n for n in got}
        return loaded


def build_speech_tokenizer(config: dict, device=None, with_encoder: bool = True):
    """The tokenizer class named by a ``speech_tokenizer/config.json``'s ``model_type``
    (vllm_omni/model_executor/models/qwen3_tts/qwen3_tts_tokenizer.py:334-379)."""
    kind = (config or {}).get("model_type", "qwen3_tts_tokenizer_12hz")
    if kind == "qwen3_tts_tokenizer_25hz":
        return Qwen3TTSTokenizer25Hz(Tokenizer25HzConfig.from_dict(config), device, with_encoder)
    if kind == "qwen3_tts_tokenizer_12hz":
        from .tokenizer_12hz import Qwen3TTSTokenizerDecoder, TokenizerDecoderConfig
        return Qwen3TTSTokenizerDecoder(TokenizerDecoderConfig.from_dict(config.get("decoder_config") or {}),
                                        torch.bfloat16 if device is not None and str(device).startswith("cuda") else torch.float32,
                                        device)
    raise ValueError(f"unknown speech tokenizer type {kind!r}")
