"""Stable Audio Open text-to-audio pipeline (vllm_omni/diffusion/models/stable_audio/
pipeline_stable_audio.py:60-575): T5 text states (padded positions zeroed) through the projection
model, two extra conditioning tokens for the start / end seconds, the Stable Audio DiT under
classifier-free guidance against an all-zero conditioning (or a negative prompt), the stochastic
DPM-Solver++ sampler on its EDM noise scale, and the Oobleck decoder to a stereo 44.1 kHz waveform
cut to [start, end) seconds.  The engine reports the result as ``final_output_type='audio'``.

Per request: ``extra_args`` ``audio_start_in_s`` (0) and ``audio_end_in_s`` (the model's full
window; ``audio_seconds`` is accepted as an alias).  The conditioning tokens do not change over the
steps, so every block's cross-attention keys / values are computed once per request.
"""
from __future__ import annotations

import json
import os

import torch
from torch import nn

from ...data import DiffusionOutput, OmniDiffusionConfig
from ...schedulers.cosine_dpm import CosineDPMSolverMultistepScheduler
from ..qwen_image.pipeline import HashTextEncoder
from ..vae.oobleck import AutoencoderOobleck, OobleckConfig
from .transformer import (StableAudioDiTConfig, StableAudioDiTModel, StableAudioProjectionConfig,
                          StableAudioProjectionModel)


class StableAudioPipeline(nn.Module):
    default_guidance = 7.0
    max_text_len = 128

    def __init__(self, od_config: OmniDiffusionConfig | None = None, transformer_config=None, vae_config=None, device=None, **_):
        super().__init__()
        self.od_config = od_config or OmniDiffusionConfig()
        dtype = self.od_config.dtype
        self.device_ = torch.device(device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu"))
        p = self.od_config.tf_model_config.to_dict()
        self.transformer = StableAudioDiTModel(transformer_config or StableAudioDiTConfig.from_dict(p), dtype, self.device_)
        tc = self.transformer.cfg
        vc = dict(vae_config or self.od_config.vae_config or {})
        vc.setdefault("decoder_input_channels", tc.out_channels)
        model = self.od_config.model
        sub = lambda name: self._read_json(model, name)
        self.vae = AutoencoderOobleck(OobleckConfig.from_dict({**vc, **sub("vae")}), torch.float32, self.device_)
        pc = {"text_encoder_dim": tc.cross_attention_input_dim, "conditioning_dim": tc.cross_attention_input_dim, **sub("projection_model")}
        self.projection_model = StableAudioProjectionModel(StableAudioProjectionConfig.from_dict(pc), dtype, self.device_)
        self.scheduler = CosineDPMSolverMultistepScheduler(**sub("scheduler"))
        self.text_encoder = HashTextEncoder(self.projection_model.config.text_encoder_dim, max_len=self.max_text_len)

    @staticmethod
    def _read_json(model, name) -> dict:
        for fn in ("config.json", "scheduler_config.json"):
            path = os.path.join(model or "", name, fn)
            if model and os.path.isfile(path):
                with open(path) as f:
                    return {k: v for k, v in json.load(f).items() if not k.startswith("_")}
        return {}

    def attach_text_encoder(self, model_path: str) -> bool:
        if not (os.path.isfile(os.path.join(model_path, "text_encoder", "config.json")) and
                os.path.isdir(os.path.join(model_path, "tokenizer"))):
            return False
        from ..text_encoders.t5 import T5PromptEncoder
        self.text_encoder = T5PromptEncoder.from_pretrained(model_path, "text_encoder", "tokenizer", self.od_config.dtype,
                                                            self.device_, max_len=self.max_text_len, zero_padding=True)
        self.text_encoder.max_len = min(self.max_text_len, int(getattr(self.text_encoder.tokenizer, "model_max_length", 128)))
        return True

    def load_weights(self, weights) -> set:
        groups = {"transformer": [], "vae": [], "projection_model": [], "text_encoder": []}
        for n, w in weights:
            comp, _, rest = n.partition(".")
            if comp in groups:
                groups[comp].append((rest, w))
        loaded = set()
        for comp, mod in (("transformer", self.transformer), ("vae", self.vae), ("projection_model", self.projection_model),
                          ("text_encoder", self.text_encoder)):
            if groups[comp] and hasattr(mod, "load_weights"):
                loaded |= {comp + "." + n for n in mod.load_weights(groups[comp])}
        return loaded

    # ------------------------------------------------------------------ conditioning
    def encode_prompt(self, texts):
        """[B, S, D] projected text states; positions of padding are zero."""
        states, mask = self.text_encoder(texts, self.device_, self.od_config.dtype, self.max_text_len)
        states = self.projection_model.project_text(states)
        return states * mask[..., None].to(states.dtype)

    @torch.no_grad()
    def forward(self, req) -> DiffusionOutput:
        sp = req.sampling_params
        tf, vae = self.transformer, self.vae
        dt_model = self.od_config.dtype
        extra = sp.extra_args or {}
        texts = [p if isinstance(p, str) else (p.get("prompt") or "") for p in req.prompts]
        negs = [None if isinstance(p, str) else p.get("negative_prompt") for p in req.prompts]
        has_neg = any(n is not None for n in negs)
        B = len(texts)
        sr, hop = vae.config.sampling_rate, vae.hop_length
        window = tf.cfg.sample_size * hop / sr
        start = float(extra.get("audio_start_in_s", 0.0))
        end = extra.get("audio_end_in_s", extra.get("audio_seconds"))
        end = window if end is None else float(end)
        if end < start:
            raise ValueError(f"audio_end_in_s={end} must not be smaller than audio_start_in_s={start}")
        if end - start > window + 1e-6:
            raise ValueError(f"requested {end - start:.2f} s of audio, the model's window is {window:.2f} s")
        scale = float(sp.guidance_scale) if sp.guidance_scale_provided else self.default_guidance
        do_cfg = scale > 1.0
        pm = self.projection_model
        text = self.encode_prompt(texts)
        dev = self.device_
        s_tok = pm.start_number_conditioner(torch.full((B,), start, device=dev)).to(text.dtype)
        e_tok = pm.end_number_conditioner(torch.full((B,), end, device=dev)).to(text.dtype)
        cond = torch.cat([text, s_tok, e_tok], dim=1)
        glob = torch.cat([s_tok, e_tok], dim=2)
        if do_cfg:                                       # unconditional branch first, as the reference batches it
            if has_neg:
                ntext = self.encode_prompt([n or "" for n in negs])
                cond = torch.cat([torch.cat([ntext, s_tok, e_tok], dim=1), cond], dim=0)
            else:
                cond = torch.cat([torch.zeros_like(cond), cond], dim=0)
            glob = torch.cat([glob, glob], dim=0)
        cross_kv = tf.conditioning(cond)
        L = int(extra.get("latent_length", tf.cfg.sample_size))
        gen = sp.generator or (torch.Generator(device="cpu").manual_seed(int(sp.seed)) if sp.seed is not None else None)
        gdev = gen.device if gen is not None else dev
        sched = self.scheduler
        ts = sched.set_timesteps(sp.num_inference_steps, device=dev)
        lat = torch.randn(B, tf.cfg.in_channels, L, generator=gen, device=gdev).to(dev, torch.float32) * sched.init_noise_sigma
        for t in ts:
            x = sched.scale_model_input(lat).to(dt_model)
            if do_cfg:
                x = torch.cat([x, x], dim=0)
            v = tf(x, t.reshape(1), global_hidden_states=glob, cross_kv=cross_kv).float()
            if do_cfg:
                v = v[:B] + scale * (v[B:] - v[:B])
            lat = sched.step(v, lat, generator=gen)
        if (sp.output_type or self.od_config.output_type) == "latent":
            return DiffusionOutput(output=lat)
        wav = vae.decode(lat).float()
        wav = wav[:, :, int(start * sr):int(end * sr)]
        return DiffusionOutput(output=[w for w in wav], metrics={"num_steps": len(ts), "sample_rate": sr})
