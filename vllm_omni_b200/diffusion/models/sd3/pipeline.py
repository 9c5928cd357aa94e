"""Stable Diffusion 3 pipeline (vllm_omni/diffusion/models/sd3/pipeline_sd3.py): MMDiT over 2x2
packed 16-channel latents, conditioning = text states [CLIP-L | CLIP-G (padded) ; T5] plus the
pooled CLIP vector, classifier-free guidance with cond/uncond in one batch, shifted flow-match
Euler schedule, 2-D AutoencoderKL."""
from __future__ import annotations

import torch

from ....ops import fused
from ...data import DiffusionOutput
from ...schedulers.flow_match_euler import FlowMatchEulerDiscreteScheduler
from ..flux.pipeline import FluxPipeline
from ..qwen_image.pipeline import pack_latents, unpack_latents
from .transformer import SD3Transformer2DModel, SD3TransformerConfig


class StableDiffusion3Pipeline(FluxPipeline):
    transformer_cls, config_cls = SD3Transformer2DModel, SD3TransformerConfig
    default_guidance = 7.0
    max_text_len = 333

    def __init__(self, od_config=None, transformer_config=None, vae_config=None, device=None, **kw):
        vc = dict(vae_config or (od_config.vae_config if od_config else {}) or {})
        vc.setdefault("scaling_factor", 1.5305)
        vc.setdefault("shift_factor", 0.0609)
        super().__init__(od_config, transformer_config, vc, device)
        self.scheduler = FlowMatchEulerDiscreteScheduler(shift=3.0)

    @torch.no_grad()
    def forward(self, req) -> DiffusionOutput:
        sp = req.sampling_params
        dt_model = self.od_config.dtype
        texts = [p if isinstance(p, str) else p.get("prompt", "") for p in req.prompts]
        negs = [(p.get("negative_prompt") if isinstance(p, dict) else None) or "" for p in req.prompts]
        H, W = sp.height or 1024, sp.width or 1024
        h, w = 2 * (H // 16), 2 * (W // 16)
        scale = float(sp.guidance_scale) if sp.guidance_scale_provided else self.default_guidance
        do_cfg = scale > 1.0
        pe, mask = self.text_encoder(texts, self.device_, dt_model, sp.max_sequence_length)
        pooled = self.pooled_encoder(texts, self.device_, dt_model)[0][:, 0]
        lens = mask.sum(1).tolist()
        B = pe.shape[0]
        if do_cfg:
            ne, nmask = self.text_encoder(negs, self.device_, dt_model, sp.max_sequence_length)
            npooled = self.pooled_encoder(negs, self.device_, dt_model)[0][:, 0]
            L = max(pe.shape[1], ne.shape[1])
            both = pe.new_zeros(2 * B, L, pe.shape[2])
            both[:B, :pe.shape[1]], both[B:, :ne.shape[1]] = pe, ne
            pe, pooled, lens = both, torch.cat([pooled, npooled]), lens + nmask.sum(1).tolist()
        gen = sp.generator or (torch.Generator(device="cpu").manual_seed(int(sp.seed)) if sp.seed is not None else None)
        C = self.transformer.cfg.in_channels // 4
        z = torch.randn(B, C, h, w, generator=gen, device=gen.device if gen is not None else self.device_)
        lat = pack_latents(z.to(self.device_, torch.float32))
        ts = self.scheduler.set_timesteps(sp.num_inference_steps, device=self.device_)
        lat_in = lat.to(dt_model)
        nb = 2 * B if do_cfg else B
        tv = torch.empty(nb, device=self.device_)
        for i in range(len(ts)):
            tv.fill_(float(self.scheduler.sigmas[i]))
            x = lat_in.repeat(2, 1, 1) if do_cfg else lat_in
            v = self.transformer(x, pe, tv, (1, h // 2, w // 2), pooled_projections=pooled, txt_seq_lens=lens)
            if do_cfg:
                fused.cfg_euler_step_(v[:B].contiguous(), v[B:].contiguous(), lat, scale, self.scheduler.dt(i), False, lat_in)
            else:
                fused.cfg_euler_step_(v.contiguous(), None, lat, 1.0, self.scheduler.dt(i), False, lat_in)
        if (sp.output_type or self.od_config.output_type) == "latent":
            return DiffusionOutput(output=lat)
        return DiffusionOutput(output=(self.vae_decode or self.vae.decode)(unpack_latents(lat, h, w)))
