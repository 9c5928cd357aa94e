"""Bagel image generation stage (vllm_omni/diffusion/models/bagel/pipeline_bagel.py:319-327):
the DiT stage of an AR -> DiT pipeline.  The upstream AR stage prefills the prompt and hands its
KV cache over through the KV transfer manager; this stage injects it as ``past_key_values`` —
every attention layer attends to [received KV | its own tokens] — instead of re-encoding the
prompt."""
from __future__ import annotations

import torch

from ....ops import fused
from ...data import DiffusionOutput
from ...schedulers.flow_match_euler import FlowMatchEulerDiscreteScheduler
from ..flux.pipeline import FluxPipeline
from ..qwen_image.pipeline import pack_latents, unpack_latents
from .transformer import BagelTransformer2DModel, BagelTransformerConfig


class BagelPipeline(FluxPipeline):
    transformer_cls, config_cls = BagelTransformer2DModel, BagelTransformerConfig
    default_guidance = 0.0

    def __init__(self, od_config=None, transformer_config=None, vae_config=None, device=None, **kw):
        tc = transformer_config or BagelTransformerConfig.from_dict(od_config.tf_model_config.to_dict() if od_config else {})
        tc.joint_attention_dim = tc.cap_feat_dim          # the text-encoder width the base class sizes its encoder by
        super().__init__(od_config, tc, vae_config, device)
        self.scheduler = FlowMatchEulerDiscreteScheduler(shift=3.0)

    @torch.no_grad()
    def forward(self, req):
        sp = req.sampling_params
        if sp.need_kv_receive and sp.past_key_values is None:
            raise RuntimeError("BagelPipeline expects the prompt KV cache from the AR stage (past_key_values); "
                               "none was received")
        texts = [p if isinstance(p, str) else p.get("prompt", "") for p in req.prompts]
        H, W = sp.height or 1024, sp.width or 1024
        h, w = 2 * (H // 16), 2 * (W // 16)
        pe, mask = self.text_encoder(texts, self.device_, self.od_config.dtype, sp.max_sequence_length)
        B = pe.shape[0]
        gen = sp.generator or (torch.Generator(device="cpu").manual_seed(int(sp.seed)) if sp.seed is not None else None)
        C = self.transformer.cfg.in_channels // 4
        z = torch.randn(B, C, h, w, generator=gen, device=gen.device if gen is not None else self.device_)
        lat = pack_latents(z.to(self.device_, torch.float32))
        ts = self.scheduler.set_timesteps(sp.num_inference_steps, device=self.device_)
        lat_in = lat.to(self.od_config.dtype)
        tv = torch.empty(B, device=self.device_)
        for i in range(len(ts)):
            tv.fill_(float(self.scheduler.sigmas[i]))
            v = self.transformer(lat_in, pe, tv, (1, h // 2, w // 2), txt_seq_lens=mask.sum(1).tolist(),
                                 past_key_values=sp.past_key_values)
            fused.cfg_euler_step_(v.contiguous(), None, lat, 1.0, self.scheduler.dt(i), False, lat_in)
        if (sp.output_type or self.od_config.output_type) == "latent":
            return DiffusionOutput(output=lat)
        return DiffusionOutput(output=(self.vae_decode or self.vae.decode)(unpack_latents(lat, h, w)))
