"""Z-Image text-to-image pipeline (vllm_omni/diffusion/models/z_image/pipeline_z_image.py:236-640).

Caption features (second-to-last hidden layer of the Qwen3 text encoder over the chat-templated
prompt) condition a single-stream DiT; latents are [B, 16, H/8, W/8] and are patchified by the
transformer's own 2x2 layout.  The network is fed ``1 - sigma`` as time and predicts the negative
velocity.  Classifier-free guidance is ``pos + s (pos - neg)`` on one 2B batch, optionally
truncated late in the schedule (``cfg_truncation``) and norm-limited (``cfg_normalization``).  The
distilled "Turbo" checkpoints run 8 steps without guidance.  VAE: the 2-D ``AutoencoderKL``; VAE
patch parallelism is allowed for this pipeline.
"""
from __future__ import annotations

import torch

from ....ops import fused
from ...data import DiffusionOutput
from ...schedulers.flow_match_euler import FlowMatchEulerDiscreteScheduler
from ..flux.pipeline import FluxPipeline
from .transformer import ZImageTransformer2DModel, ZImageTransformerConfig


class ZImagePipeline(FluxPipeline):
    transformer_cls, config_cls = ZImageTransformer2DModel, ZImageTransformerConfig
    default_guidance = 0.0
    max_text_len = 512

    def __init__(self, od_config=None, transformer_config=None, vae_config=None, device=None, **kw):
        tc = transformer_config or ZImageTransformerConfig.from_dict((od_config.tf_model_config.to_dict() if od_config else {}))
        tc.joint_attention_dim = tc.cap_feat_dim          # the text-encoder width the base class sizes its encoder by
        vc = dict(vae_config or (od_config.vae_config if od_config else {}) or {})
        vc.setdefault("latent_channels", tc.in_channels)
        super().__init__(od_config, tc, vc, device)
        self.scheduler = FlowMatchEulerDiscreteScheduler(shift=3.0)

    def attach_text_encoder(self, model_path: str) -> bool:
        import os
        if not (os.path.isfile(os.path.join(model_path, "text_encoder", "config.json")) and
                os.path.isdir(os.path.join(model_path, "tokenizer"))):
            return False
        from .text_encoder import QwenCaptionEncoder
        self.text_encoder = QwenCaptionEncoder.from_pretrained(model_path, self.od_config.dtype, self.device_)
        return True

    def load_weights(self, weights) -> set:
        ew, rest = [], []
        for n, w in weights:
            (ew if n.startswith("text_encoder.") else rest).append((n, w))
        loaded = super().load_weights(rest)
        if ew and hasattr(self.text_encoder, "load_weights"):
            loaded |= {"text_encoder." + n for n in self.text_encoder.load_weights([(n[len("text_encoder."):], w) for n, w in ew])}
        return loaded

    @torch.no_grad()
    def forward(self, req):
        sp = req.sampling_params
        tf = self.transformer
        dt_model = self.od_config.dtype
        texts = [p if isinstance(p, str) else p.get("prompt", "") for p in req.prompts]
        negs = [(p.get("negative_prompt") if isinstance(p, dict) else None) or "" for p in req.prompts]
        H, W = sp.height or 1024, sp.width or 1024
        h, w = 2 * (H // 16), 2 * (W // 16)
        scale = float(sp.guidance_scale) if sp.guidance_scale_provided else self.default_guidance
        do_cfg = scale > 1.0
        extra = sp.extra_args or {}
        cfg_trunc = float(extra.get("cfg_truncation", 1.0))
        cfg_norm = float(extra.get("cfg_normalization", 0.0) or 0.0)
        pe, mask = self.text_encoder(texts, self.device_, dt_model, sp.max_sequence_length)
        lens = mask.sum(1).tolist()
        B = pe.shape[0]
        if do_cfg:
            ne, nmask = self.text_encoder(negs, self.device_, dt_model, sp.max_sequence_length)
            L = max(pe.shape[1], ne.shape[1])
            both = pe.new_zeros(2 * B, L, pe.shape[2])
            both[:B, :pe.shape[1]], both[B:, :ne.shape[1]] = pe, ne
            lens2 = lens + nmask.sum(1).tolist()
        gen = sp.generator or (torch.Generator(device="cpu").manual_seed(int(sp.seed)) if sp.seed is not None else None)
        C = tf.cfg.in_channels
        z = torch.randn(B, C, h, w, generator=gen, device=gen.device if gen is not None else self.device_)
        lat = tf.patchify(z.to(self.device_, torch.float32)).contiguous()          # fp32 master copy, patch layout
        steps = sp.num_inference_steps if sp.num_inference_steps != 50 else 8
        ts = self.scheduler.set_timesteps(steps, device=self.device_)
        grid = (1, h // 2, w // 2)
        lat_in = lat.to(dt_model)
        for i in range(len(ts)):
            sigma = float(self.scheduler.sigmas[i])
            t_in = 1.0 - sigma                                  # the network's time runs from 0 (noise) to 1 (clean)
            cfg_now = do_cfg and not (cfg_trunc <= 1.0 and t_in > cfg_trunc)
            if cfg_now:
                out = tf(lat_in.repeat(2, 1, 1), both, torch.full((2 * B,), t_in, device=self.device_), grid, txt_seq_lens=lens2)
                pos, neg = out[:B].float(), out[B:].float()
                pred = pos + scale * (pos - neg)
                if cfg_norm > 0:
                    flat = lambda t: t.reshape(B, -1)
                    lim = torch.linalg.vector_norm(flat(pos), dim=1) * cfg_norm
                    new = torch.linalg.vector_norm(flat(pred), dim=1)
                    pred = pred * torch.where(new > lim, lim / new.clamp_min(1e-12), torch.ones_like(new))[:, None, None]
                lat.add_(pred, alpha=-self.scheduler.dt(i))     # the model predicts the negative velocity
                lat_in = lat.to(dt_model)
            else:
                v = tf(lat_in, pe, torch.full((B,), t_in, device=self.device_), grid, txt_seq_lens=lens)
                fused.cfg_euler_step_(v.contiguous(), None, lat, 1.0, -self.scheduler.dt(i), False, lat_in)
        z = tf.unpatchify(lat, 1, h, w)[:, :, 0]
        if (sp.output_type or self.od_config.output_type) == "latent":
            return DiffusionOutput(output=z)
        return DiffusionOutput(output=(self.vae_decode or self.vae.decode)(z))
