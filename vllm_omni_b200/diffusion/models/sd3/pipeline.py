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


class SD3PromptEncoder:
    """SD3 conditioning from its three encoders: the penultimate states of CLIP-L and CLIP-G side by
    side, zero-padded to the T5 width and followed by the T5 states along the sequence; the pooled
    vector is the two projected CLIP end-of-text vectors side by side.  A missing T5 (the checkpoint
    may ship without it) contributes zero states, as in diffusers."""

    def __init__(self, clip_l, clip_g, t5, joint_dim: int, t5_len: int = 256):
        self.clip_l, self.clip_g, self.t5, self.joint_dim, self.t5_len = clip_l, clip_g, t5, joint_dim, t5_len
        self._key, self._val = None, None

    def _encode(self, texts, device, dtype, max_len):
        key = (tuple(texts), str(device), dtype, max_len)
        if key != self._key:
            _, pool_l, pen_l = self.clip_l.encode(texts, device)
            _, pool_g, pen_g = self.clip_g.encode(texts, device)
            clip = torch.cat([pen_l, pen_g], dim=-1)
            clip = torch.nn.functional.pad(clip, (0, self.joint_dim - clip.shape[-1]))
            L = min(int(max_len or self.t5_len), self.t5_len)
            if self.t5 is not None:
                t5, _ = self.t5(texts, device, None, L)
            else:
                t5 = clip.new_zeros(clip.shape[0], L, self.joint_dim)
            self._key = key
            self._val = (torch.cat([clip, t5.to(clip.dtype)], dim=1).to(dtype), torch.cat([pool_l, pool_g], dim=-1).to(dtype))
        return self._val

    def __call__(self, texts, device, dtype=None, max_len=None):
        pe, _ = self._encode(list(texts), device, dtype, max_len)
        return pe, torch.ones(pe.shape[:2], dtype=torch.long, device=pe.device)

    def pooled(self, texts, device, dtype=None, max_len=None):
        pooled = self._encode(list(texts), device, dtype, max_len)[1]
        return pooled[:, None], None

    def load_component(self, comp: str, weights) -> set:
        enc = {"text_encoder": self.clip_l, "text_encoder_2": self.clip_g, "text_encoder_3": self.t5}.get(comp)
        return enc.load_weights(weights) if enc is not None else set()


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

    def attach_text_encoder(self, model_path: str) -> bool:
        """``text_encoder/`` + ``text_encoder_2/`` (CLIP-L and CLIP-G with projection) and, when present,
        ``text_encoder_3/`` (T5) with ``tokenizer*/`` replace the seeded stand-ins."""
        import os
        from ..text_encoders.clip import CLIPPromptEncoder
        from ..text_encoders.t5 import T5PromptEncoder
        has = lambda enc, tok: (os.path.isfile(os.path.join(model_path, enc, "config.json")) and
                                os.path.isdir(os.path.join(model_path, tok)))
        if not (has("text_encoder", "tokenizer") and has("text_encoder_2", "tokenizer_2")):
            return False
        dt, dev = self.od_config.dtype, self.device_
        clip_l = CLIPPromptEncoder.from_pretrained(model_path, "text_encoder", "tokenizer", dt, dev, with_projection=True)
        clip_g = CLIPPromptEncoder.from_pretrained(model_path, "text_encoder_2", "tokenizer_2", dt, dev, with_projection=True)
        t5 = T5PromptEncoder.from_pretrained(model_path, "text_encoder_3", "tokenizer_3", dt, dev, max_len=256) \
            if has("text_encoder_3", "tokenizer_3") else None
        enc = SD3PromptEncoder(clip_l, clip_g, t5, self.transformer.cfg.joint_attention_dim)
        self.text_encoder, self.pooled_encoder = enc, enc.pooled
        return True

    def load_weights(self, weights) -> set:
        rest, enc = [], {"text_encoder": [], "text_encoder_2": [], "text_encoder_3": []}
        for n, w in weights:
            comp, _, tail = n.partition(".")
            if comp in enc:
                enc[comp].append((tail, w))
            else:
                rest.append((n, w))
        loaded = super().load_weights(rest)
        if isinstance(self.text_encoder, SD3PromptEncoder):
            for comp, ws in enc.items():
                if ws:
                    loaded |= {comp + "." + n for n in self.text_encoder.load_component(comp, ws)}
        return loaded

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
        cfg_par = do_cfg and self.cfg_exchange is not None       # one guidance branch per rank instead of a doubled batch
        if do_cfg:
            ne, nmask = self.text_encoder(negs, self.device_, dt_model, sp.max_sequence_length)
            npooled = self.pooled_encoder(negs, self.device_, dt_model)[0][:, 0]
            if cfg_par:
                if self.cfg_exchange.is_negative_rank:
                    pe, pooled, lens = ne, npooled, nmask.sum(1).tolist()
            else:
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
        nb = 2 * B if (do_cfg and not cfg_par) else B
        tv = torch.empty(nb, device=self.device_)
        for i in range(len(ts)):
            tv.fill_(float(self.scheduler.sigmas[i]))
            x = lat_in.repeat(2, 1, 1) if (do_cfg and not cfg_par) else lat_in
            v = self.transformer(x, pe, tv, (1, h // 2, w // 2), pooled_projections=pooled, txt_seq_lens=lens)
            if cfg_par:
                self.cfg_exchange.step(v.contiguous(), lat, scale, self.scheduler.dt(i), False, lat_in)
            elif do_cfg:
                fused.cfg_euler_step_(v[:B].contiguous(), v[B:].contiguous(), lat, scale, self.scheduler.dt(i), False, lat_in)
            else:
                fused.cfg_euler_step_(v.contiguous(), None, lat, 1.0, self.scheduler.dt(i), False, lat_in)
        if (sp.output_type or self.od_config.output_type) == "latent":
            return DiffusionOutput(output=lat)
        return DiffusionOutput(output=(self.vae_decode or self.vae.decode)(unpack_latents(lat, h, w)))
