"""Z-Image pipeline (vllm_omni/diffusion/models/z_image/pipeline_z_image.py): few-step distilled
text-to-image, CFG optional, VAE patch parallelism allowed."""
from __future__ import annotations

import numpy as np
import torch

from ....ops import fused
from ...data import DiffusionOutput
from ...schedulers.flow_match_euler import FlowMatchEulerDiscreteScheduler
from ..flux.pipeline import FluxPipeline
from ..qwen_image.pipeline import pack_latents, unpack_latents
from .transformer import ZImageTransformer2DModel, ZImageTransformerConfig


class ZImagePipeline(FluxPipeline):
    transformer_cls, config_cls = ZImageTransformer2DModel, ZImageTransformerConfig
    default_guidance = 0.0

    def __init__(self, od_config=None, transformer_config=None, vae_config=None, device=None, **kw):
        tc = transformer_config or ZImageTransformerConfig.from_dict((od_config.tf_model_config.to_dict() if od_config else {}))
        tc.joint_attention_dim = tc.cap_feat_dim          # the text-encoder width the base class sizes its encoder by
        super().__init__(od_config, tc, vae_config, device)
        self.scheduler = FlowMatchEulerDiscreteScheduler(shift=3.0)

    @torch.no_grad()
    def forward(self, req):
        sp = req.sampling_params
        texts = [p if isinstance(p, str) else p.get("prompt", "") for p in req.prompts]
        H, W = sp.height or 1024, sp.width or 1024
        h, w = 2 * (H // 16), 2 * (W // 16)
        pe, mask = self.text_encoder(texts, self.device_, self.od_config.dtype, sp.max_sequence_length)
        B = pe.shape[0]
        gen = sp.generator or (torch.Generator(device="cpu").manual_seed(int(sp.seed)) if sp.seed is not None else None)
        C = self.transformer.cfg.in_channels // 4
        z = torch.randn(B, C, h, w, generator=gen, device=gen.device if gen is not None else self.device_)
        lat = pack_latents(z.to(self.device_, torch.float32))
        steps = sp.num_inference_steps if sp.num_inference_steps != 50 else 8
        ts = self.scheduler.set_timesteps(steps, device=self.device_)
        lat_in = lat.to(self.od_config.dtype)
        tv = torch.empty(B, device=self.device_)
        pkv = sp.past_key_values
        for i in range(len(ts)):
            tv.fill_(float(self.scheduler.sigmas[i]))
            v = self.transformer(lat_in, pe, tv, (1, h // 2, w // 2), txt_seq_lens=mask.sum(1).tolist(),
                                 past_key_values=pkv)
            fused.cfg_euler_step_(v.contiguous(), None, lat, 1.0, self.scheduler.dt(i), False, lat_in)
        if (sp.output_type or self.od_config.output_type) == "latent":
            return DiffusionOutput(output=lat)
        return DiffusionOutput(output=(self.vae_decode or self.vae.decode)(unpack_latents(lat, h, w)))
