"""GLM-Image pipeline (vllm_omni/diffusion/models/glm_image/pipeline_glm_image.py:253-960): an AR
vision-language model first writes a grid of prior VQ tokens for the picture; the DiT then denoises
latents conditioned on those tokens (one per 2x2 latent patch), on glyph-text states and on the
target size.  Classifier-free guidance runs the DiT twice per step, the second time with the prior
tokens dropped and the negative text; under CFG-parallel the two passes run on two ranks (the
reference carries an inline copy of that exchange, :713-724; here it is the shared mechanism).

In a multi-stage deployment the AR stage hands ``prior_token_ids`` over in
``sampling_params.extra_args``; without them (random-weight runs) a seeded stand-in grid is used.
Editing: the condition images pass once through the DiT in "write" mode, which fills a per-layer
key / value cache that every denoising step reads.
"""
from __future__ import annotations

import hashlib

import torch
from torch import nn

from ...data import DiffusionOutput, OmniDiffusionConfig
from ...schedulers.flow_match_euler import FlowMatchEulerDiscreteScheduler
from ..qwen_image.pipeline import HashTextEncoder
from ..vae import build_vae
from .transformer import GlmImageKVCache, GlmImageTransformer2DModel, GlmImageTransformerConfig


class GlmImagePipeline(nn.Module):
    vae_scale_factor = 8

    def __init__(self, od_config: OmniDiffusionConfig | None = None, transformer_config=None, vae_config=None, device=None, **_):
        super().__init__()
        self.od_config = od_config or OmniDiffusionConfig()
        dtype = self.od_config.dtype
        self.device_ = torch.device(device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu"))
        tc = transformer_config or GlmImageTransformerConfig.from_dict(self.od_config.tf_model_config.to_dict())
        self.transformer = GlmImageTransformer2DModel(tc, dtype=dtype, device=self.device_)
        vc = dict(vae_config or self.od_config.vae_config or {})
        vc.setdefault("latent_channels", tc.in_channels)
        self.vae = build_vae(vc, "kl", with_encoder=True).to(device=self.device_, dtype=dtype)
        self.scheduler = FlowMatchEulerDiscreteScheduler(shift=1.0)
        self.text_encoder = HashTextEncoder(tc.text_embed_dim, max_len=64)
        self.vae_decode = None
        self.cfg_exchange = None

    def _prior_tokens(self, text: str, n: int, extra: dict):
        ids = extra.get("prior_token_ids")
        if ids is not None:
            ids = torch.as_tensor(ids, dtype=torch.long).reshape(1, -1)
            if ids.shape[1] != n:
                raise ValueError(f"prior_token_ids has {ids.shape[1]} entries, the latent grid has {n} patches")
            return ids.to(self.device_)
        seed = int.from_bytes(hashlib.sha256(text.encode()).digest()[:8], "little") % (2 ** 31)
        g = torch.Generator().manual_seed(seed)
        V = self.transformer.cfg.prior_vq_quantizer_codebook_size
        return torch.randint(0, V, (1, n), generator=g).to(self.device_)

    @torch.no_grad()
    def forward(self, req) -> DiffusionOutput:
        sp = req.sampling_params
        tf, dt_model = self.transformer, self.od_config.dtype
        p = req.prompts[0]
        text = p if isinstance(p, str) else p.get("prompt", "")
        neg = (p.get("negative_prompt") if isinstance(p, dict) else None) or ""
        extra = sp.extra_args or {}
        H, W = sp.height or 1024, sp.width or 1024
        h, w = 2 * (H // 16), 2 * (W // 16)
        scale = float(sp.guidance_scale) if sp.guidance_scale_provided else 1.5
        do_cfg = scale > 1.0
        pe, mask = self.text_encoder([text], self.device_, dt_model)
        pe = pe[:, :int(mask.sum())]
        ne = None
        if do_cfg:
            ne, nmask = self.text_encoder([neg], self.device_, dt_model)
            ne = ne[:, :int(nmask.sum())]
        n_patch = (h // 2) * (w // 2)
        prior = self._prior_tokens(text, n_patch, extra)
        keep, drop = torch.zeros_like(prior, dtype=torch.bool), torch.ones_like(prior, dtype=torch.bool)
        target = torch.tensor([[H, W]], dtype=torch.float32, device=self.device_)
        crop = torch.zeros(1, 2, device=self.device_)
        cache = None
        mm = (p.get("multi_modal_data") or {}) if isinstance(p, dict) else {}
        cond_images = mm.get("image_tensor") or []
        if cond_images:                                   # editing: cache the condition images' keys / values
            cache = GlmImageKVCache(tf.cfg.num_layers)
            cache.mode = "write"
            cond_prior = extra.get("prior_token_image_ids") or [None] * len(cond_images)
            for im, cp in zip(cond_images, cond_prior):
                x = im.to(self.device_, dt_model)[None]
                x = torch.nn.functional.interpolate(x.float(), size=(H, W), mode="bilinear", align_corners=False).to(dt_model)
                z = self.vae.encode(x).to(dt_model)
                ids = self._prior_tokens(text + "#cond", n_patch, {"prior_token_ids": cp} if cp is not None else {})
                tf(z, pe, ids, torch.zeros_like(ids, dtype=torch.bool), torch.zeros(1, device=self.device_), target, crop,
                   kv_cache=cache)
            cache.mode = "read"
        gen = sp.generator or (torch.Generator(device="cpu").manual_seed(int(sp.seed)) if sp.seed is not None else None)
        C = tf.cfg.in_channels
        lat = torch.randn(1, C, h, w, generator=gen, device=gen.device if gen is not None else self.device_).to(self.device_, torch.float32)
        ts = self.scheduler.set_timesteps(sp.num_inference_steps, device=self.device_)
        for i in range(len(ts)):
            t = torch.full((1,), float(self.scheduler.sigmas[i]) * 1000.0 - 1.0, device=self.device_)
            x = lat.to(dt_model)
            v = tf(x, pe, prior, keep, t, target, crop, kv_cache=cache).float()
            if do_cfg:
                vu = tf(x, ne, prior, drop, t, target, crop, kv_cache=cache).float()
                v = vu + scale * (v - vu)
            lat = lat + self.scheduler.dt(i) * v
        if (sp.output_type or self.od_config.output_type) == "latent":
            return DiffusionOutput(output=lat)
        return DiffusionOutput(output=(self.vae_decode or self.vae.decode)(lat))

    def load_weights(self, weights) -> set:
        tw, vw = [], []
        for n, w in weights:
            if n.startswith("transformer."):
                tw.append((n[len("transformer."):], w))
            elif n.startswith("vae."):
                vw.append((n[len("vae."):], w))
        loaded = {"transformer." + n for n in self.transformer.load_weights(tw)}
        loaded |= {"vae." + n for n in self.vae.load_weights(vw)}
        return loaded
