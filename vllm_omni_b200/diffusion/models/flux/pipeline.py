"""FLUX text-to-image pipeline
(vllm_omni/diffusion/models/flux/pipeline_flux.py): guidance-distilled (the
guidance scale is an input of the network, one transformer call per step), T5 states +
pooled CLIP vector, 2x2 packed latents, shifted flow-match Euler schedule."""
from __future__ import annotations

import numpy as np
import torch
from torch import nn

from ....ops import fused
from ...data import DiffusionOutput, OmniDiffusionConfig
from ...request import OmniDiffusionRequest
from ...schedulers.flow_match_euler import FlowMatchEulerDiscreteScheduler, calculate_shift
from ..qwen_image.pipeline import HashTextEncoder, pack_latents, unpack_latents
from ..vae import build_vae
from .transformer import FluxTransformer2DModel, FluxTransformerConfig

FLUX_SCHEDULER = dict(num_train_timesteps=1000, shift=3.0, use_dynamic_shifting=True, base_shift=0.5, max_shift=1.15,
                      base_image_seq_len=256, max_image_seq_len=4096)


class FluxPipeline(nn.Module):
    vae_scale_factor = 8
    transformer_cls, config_cls = FluxTransformer2DModel, FluxTransformerConfig
    default_guidance = 3.5
    max_text_len = 512
    # FLUX.1 is guidance-distilled (the scale is an input of the network).  The FLUX-family members without a
    # guidance embedding (LongCat-Image, Ovis-Image) run true classifier-free guidance against a negative prompt:
    true_cfg = False
    cfg_renorm_clamp = False            # rescale the guided velocity per token to at most the conditional one's norm
    needs_vae_encoder = False           # editing pipelines encode their input image

    def __init__(self, od_config: OmniDiffusionConfig | None = None, transformer_config=None, vae_config=None,
                 device=None, **_):
        super().__init__()
        self.od_config = od_config or OmniDiffusionConfig()
        dtype = self.od_config.dtype
        self.device_ = torch.device(device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu"))
        tcfg = transformer_config or self.config_cls.from_dict(self.od_config.tf_model_config.to_dict())
        self.transformer = self.transformer_cls(tcfg, dtype=dtype, device=self.device_)
        self.vae = build_vae(vae_config or self.od_config.vae_config, "kl",
                             with_encoder=self.needs_vae_encoder).to(device=self.device_, dtype=dtype)
        self.vae.use_tiling = self.od_config.vae_use_tiling
        self.scheduler = FlowMatchEulerDiscreteScheduler(**FLUX_SCHEDULER)
        self.text_encoder = HashTextEncoder(tcfg.joint_attention_dim, max_len=self.max_text_len)
        self.pooled_encoder = HashTextEncoder(getattr(tcfg, "pooled_projection_dim", 768), max_len=1)
        self.vae_decode = None
        self.cfg_exchange = None        # set by CFG-parallel

    def condition_latents(self, req: OmniDiffusionRequest, B: int, h: int, w: int):
        """Packed latents [B, k*S_img, 4C] of conditioning images that ride along with the noise rows
        (editing pipelines), or None."""
        return None

    def _guided(self, v, vn, scale, renorm_min=0.0):
        out = vn.float() + scale * (v.float() - vn.float())
        if self.cfg_renorm_clamp:
            out = out * (v.float().norm(dim=-1, keepdim=True) / (out.norm(dim=-1, keepdim=True) + 1e-8)).clamp(min=renorm_min, max=1.0)
        return out

    @torch.no_grad()
    def forward(self, req: OmniDiffusionRequest) -> DiffusionOutput:
        sp = req.sampling_params
        texts = [p if isinstance(p, str) else p.get("prompt", "") for p in req.prompts]
        n = sp.num_outputs_per_prompt
        H, W = sp.height or 1024, sp.width or 1024
        h, w = 2 * (H // 16), 2 * (W // 16)
        pes = [p.get("prompt_embeds") if isinstance(p, dict) else None for p in req.prompts]
        if all(e is not None for e in pes):
            pe = torch.stack([e.reshape(-1, e.shape[-1]) for e in pes]).to(self.device_, self.od_config.dtype)
            lens = [pe.shape[1]] * pe.shape[0]
        else:
            pe, mask = self.text_encoder(texts, self.device_, self.od_config.dtype, sp.max_sequence_length)
            lens = mask.sum(1).tolist()
        pooled = self.pooled_encoder(texts, self.device_, self.od_config.dtype)[0][:, 0]
        scale = float(sp.guidance_scale if sp.guidance_scale_provided else self.default_guidance)
        do_cfg = self.true_cfg and scale > 1.0
        ne = nlens = None
        if do_cfg:
            negs = [(p.get("negative_prompt") if isinstance(p, dict) else None) or "" for p in req.prompts]
            ne, nmask = self.text_encoder(negs, self.device_, self.od_config.dtype, sp.max_sequence_length)
            nlens = nmask.sum(1).tolist()
        if n > 1:
            pe, pooled = pe.repeat_interleave(n, 0), pooled.repeat_interleave(n, 0)
            lens = [l for l in lens for _ in range(n)]
            if do_cfg:
                ne, nlens = ne.repeat_interleave(n, 0), [l for l in nlens for _ in range(n)]
        B = pe.shape[0]
        gen = sp.generator
        if gen is None and sp.seed is not None:
            gen = torch.Generator(device="cpu").manual_seed(int(sp.seed))
        C = self.transformer.cfg.in_channels // 4
        z = torch.randn(B, C, h, w, generator=gen, device=gen.device if gen is not None else self.device_)
        lat = pack_latents(z.to(self.device_, torch.float32))
        sig = np.linspace(1.0, 1 / sp.num_inference_steps, sp.num_inference_steps) if sp.sigmas is None else sp.sigmas
        c = self.scheduler.config
        mu = calculate_shift(lat.shape[1], c["base_image_seq_len"], c["max_image_seq_len"], c["base_shift"], c["max_shift"])
        ts = self.scheduler.set_timesteps(sigmas=sig, mu=mu, device=self.device_)
        guidance = torch.full((B,), scale, device=self.device_)
        lat_in = lat.to(self.od_config.dtype)
        tv = torch.empty(B, device=self.device_)
        S_img = lat.shape[1]
        cond = self.condition_latents(req, B, h, w)
        frames = 1 if cond is None else 1 + cond.shape[1] // S_img
        for i in range(len(ts)):
            tv.fill_(float(self.scheduler.sigmas[i]))

            def call(enc, ln, branch=0):
                x = lat_in if cond is None else torch.cat([lat_in, cond.to(lat_in.dtype)], dim=1)
                v = self.transformer(x, enc, tv, (frames, h // 2, w // 2), pooled_projections=pooled,
                                     guidance=guidance, txt_seq_lens=ln, branch=branch)
                return v if cond is None else v[:, :S_img].contiguous()      # only the noise rows are stepped
            dt = self.scheduler.dt(i)
            if do_cfg and self.cfg_exchange is not None:     # one guidance branch per rank
                mine = call(ne, nlens) if self.cfg_exchange.is_negative_rank else call(pe, lens)
                if self.cfg_renorm_clamp:
                    both = self.cfg_exchange.group.all_gather(mine.contiguous(), separate_tensors=True)
                    fused.cfg_euler_step_(self._guided(both[0], both[1], scale).to(mine.dtype).contiguous(), None, lat, 1.0, dt,
                                          False, lat_in)
                else:
                    self.cfg_exchange.step(mine.contiguous(), lat, scale, dt, False, lat_in)
            elif do_cfg:
                v, vn = call(pe, lens), call(ne, nlens, 1)
                if self.cfg_renorm_clamp:
                    fused.cfg_euler_step_(self._guided(v, vn, scale).to(v.dtype).contiguous(), None, lat, 1.0, dt, False, lat_in)
                else:
                    fused.cfg_euler_step_(v.contiguous(), vn.contiguous(), lat, scale, dt, False, lat_in)
            else:
                fused.cfg_euler_step_(call(pe, lens).contiguous(), None, lat, 1.0, dt, False, lat_in)
        if (sp.output_type or self.od_config.output_type) == "latent":
            return DiffusionOutput(output=lat)
        img = (self.vae_decode or self.vae.decode)(unpack_latents(lat, h, w))
        return DiffusionOutput(output=img, metrics={"num_steps": len(ts), "batch": B})

    # sub-folder of the checkpoint -> attribute that holds its encoder (CLIP: pooled vector, T5: states)
    encoder_slots = {"text_encoder": "pooled_encoder", "text_encoder_2": "text_encoder"}

    def attach_text_encoder(self, model_path: str) -> bool:
        """``text_encoder/`` (CLIP, pooled vector) and ``text_encoder_2/`` (T5 states) with their
        tokenizers replace the seeded stand-ins when the checkpoint has them."""
        import os
        from ..text_encoders.clip import CLIPPromptEncoder
        from ..text_encoders.t5 import T5PromptEncoder
        import json

        def has(enc, tok, kind):                     # the sub-folder holds an encoder of that family, with a tokenizer
            path = os.path.join(model_path, enc, "config.json")
            if not (os.path.isfile(path) and os.path.isdir(os.path.join(model_path, tok))):
                return False
            with open(path) as f:
                d = json.load(f)
            return kind in (d.get("model_type") or "") or any(kind in a.lower() for a in d.get("architectures") or [])
        got = False
        if has("text_encoder", "tokenizer", "clip"):
            self.pooled_encoder = CLIPPromptEncoder.from_pretrained(model_path, "text_encoder", "tokenizer",
                                                                    self.od_config.dtype, self.device_)
            got = True
        if has("text_encoder_2", "tokenizer_2", "t5"):
            self.text_encoder = T5PromptEncoder.from_pretrained(model_path, "text_encoder_2", "tokenizer_2",
                                                                self.od_config.dtype, self.device_, max_len=self.max_text_len)
            got = True
        return got

    def load_weights(self, weights) -> set:
        """diffusers sub-folder prefixes ``transformer.`` / ``vae.`` / ``text_encoder*.``."""
        groups: dict[str, list] = {"transformer": [], "vae": []}
        groups.update({k: [] for k in self.encoder_slots})
        for n, w in weights:
            comp, _, rest = n.partition(".")
            if comp in groups:
                groups[comp].append((rest, w))
        loaded = {"transformer." + n for n in self.transformer.load_weights(groups["transformer"])}
        if groups["vae"] and hasattr(self.vae, "load_weights"):
            loaded |= {"vae." + n for n in self.vae.load_weights(groups["vae"])}
        for comp, attr in self.encoder_slots.items():
            enc = getattr(self, attr, None)
            if groups[comp] and hasattr(enc, "load_weights"):
                loaded |= {comp + "." + n for n in enc.load_weights(groups[comp])}
        return loaded
