"""Qwen-Image editing pipelines (vllm_omni/diffusion/models/qwen_image/pipeline_qwen_image_edit*.py,
pipeline_qwen_image_layered.py).

Edit: the input image is VAE-encoded, packed like the noise latents and appended to the image
token sequence; the transformer sees [noise tokens | condition tokens] (condition image at
frame index 1 in RoPE) and only the noise part of its output is used.  Edit-Plus takes several
condition images.  Layered generates ``layers`` RGBA-style layers as extra frames of one
sequence.  Without a VAE encoder checkpoint the condition latents come from this module's own
(randomly initialised) encoder, which keeps the data flow identical.
"""
from __future__ import annotations

import torch

from ....ops import fused
from ...data import DiffusionOutput
from ..vae.autoencoder_kl_qwenimage import AutoencoderKLQwenImage2d
from .pipeline import QwenImagePipeline, pack_latents, unpack_latents


class QwenImageEditPipeline(QwenImagePipeline):
    max_condition_images = 1
    vl_image_area = 1024 * 1024        # the condition image is shown to the prompt encoder at about this many pixels
    picture_prefix = False             # Edit-Plus numbers its images: "Picture 1: <image>Picture 2: <image>..."

    def __init__(self, od_config=None, transformer_config=None, vae_config=None, device=None, **kw):
        super().__init__(od_config, transformer_config, vae_config, device)
        enc = AutoencoderKLQwenImage2d(self.vae.cfg, with_encoder=True)
        self.vae.encoder = enc.encoder.to(self.device_, self.od_config.dtype)
        self.vae.quant_conv = enc.quant_conv.to(self.device_, self.od_config.dtype)

    def attach_text_encoder(self, model_path: str) -> bool:
        """Edit pipelines need the vision tower of the Qwen2.5-VL prompt encoder as well."""
        import os
        if not (os.path.isfile(os.path.join(model_path, "text_encoder", "config.json")) and
                os.path.isdir(os.path.join(model_path, "tokenizer"))):
            return False
        from .text_encoder import QwenVLTextEncoder
        self.text_encoder = QwenVLTextEncoder.from_pretrained(model_path, self.od_config.dtype, self.device_, with_vision=True)
        return True

    def encode_edit_prompt(self, texts, images, max_sequence_length=None):
        """Instruction + condition images through the vision-language prompt encoder; the stand-in
        encoder of random-weight runs sees the text only."""
        enc = self.text_encoder
        if getattr(enc, "visual", None) is None or not any(images):
            return self.encode_prompt(texts, max_sequence_length=max_sequence_length)
        from .text_encoder import IMAGE_SLOT
        import math
        import torch.nn.functional as F
        shown, prompts = [], []
        for text, ims in zip(texts, images):
            row = []
            for im in ims:
                r = im.shape[-1] / im.shape[-2]
                W = round(math.sqrt(self.vl_image_area * r) / 32) * 32
                H = round(W / r / 32) * 32
                row.append(F.interpolate(im[None].float(), size=(max(32, H), max(32, W)), mode="bicubic", align_corners=False,
                                         antialias=True)[0].clamp(0, 1))
            shown.append(row)
            slots = "".join((f"Picture {i + 1}: " if self.picture_prefix else "") + IMAGE_SLOT for i in range(len(row)))
            prompts.append(slots + text)
        return enc.encode_with_images(prompts, shown, self.device_, self.od_config.dtype, max_sequence_length=max_sequence_length)

    def _condition_latents(self, prompt, h, w):
        mm = (prompt.get("multi_modal_data") or {}) if isinstance(prompt, dict) else {}
        imgs = mm.get("image_tensor") or []
        out = []
        for im in imgs[: self.max_condition_images]:
            x = im.to(self.device_, self.od_config.dtype)[None]
            x = torch.nn.functional.interpolate(x.float(), size=(h * 8, w * 8), mode="bilinear",
                                                align_corners=False).to(self.od_config.dtype)
            z = self.vae.encode(x)                                  # [1, 16, h, w]
            out.append(pack_latents(z.float()))
        return out

    @torch.no_grad()
    def forward(self, req) -> DiffusionOutput:
        sp = req.sampling_params
        p = req.prompts[0]
        H = sp.height or self.default_sample_size * self.vae_scale_factor
        W = sp.width or self.default_sample_size * self.vae_scale_factor
        h, w = 2 * (H // 16), 2 * (W // 16)
        conds = self._condition_latents(p, h, w)
        if not conds:
            return super().forward(req)
        text = p.get("prompt", "") if isinstance(p, dict) else p
        neg = p.get("negative_prompt") if isinstance(p, dict) else None
        mm = (p.get("multi_modal_data") or {}) if isinstance(p, dict) else {}
        shown = [list((mm.get("image_tensor") or [])[: self.max_condition_images])]
        pe, pm = self.encode_edit_prompt([text], shown, sp.max_sequence_length)
        true_cfg = sp.true_cfg_scale if sp.true_cfg_scale is not None else (sp.guidance_scale or 1.0)
        do_cfg = true_cfg > 1 and neg is not None
        if do_cfg:
            ne, nm = self.encode_edit_prompt([neg], shown, sp.max_sequence_length)
            L = max(pe.shape[1], ne.shape[1])
            enc = torch.zeros(2, L, pe.shape[2], dtype=pe.dtype, device=pe.device)
            enc[0, :pe.shape[1]], enc[1, :ne.shape[1]] = pe[0], ne[0]
            lens = [int(pm.sum()), int(nm.sum())]
        else:
            enc, lens = pe, [int(pm.sum())]
        gen = sp.generator or (torch.Generator(device="cpu").manual_seed(int(sp.seed)) if sp.seed is not None else None)
        lat, h, w = self.prepare_latents(1, H, W, gen, sp.latents)
        S = lat.shape[1]
        cond = torch.cat(conds, dim=1).to(self.od_config.dtype)
        shapes = [(1, h // 2, w // 2)] * (1 + len(conds))
        ts = self.prepare_timesteps(sp.num_inference_steps, sp.sigmas, S)
        nb = enc.shape[0]
        tv = torch.empty(nb, device=self.device_)
        lat_lp = lat.to(self.od_config.dtype)
        for i in range(len(ts)):
            tv.fill_(float(self.scheduler.sigmas[i]))
            x = torch.cat([lat_lp, cond], dim=1).expand(nb, -1, -1).contiguous()
            v = self.transformer(x, enc, tv, shapes, txt_seq_lens=lens)[:, :S].contiguous()
            if do_cfg:
                fused.cfg_euler_step_(v[:1], v[1:], lat, float(true_cfg), self.scheduler.dt(i), True, lat_lp)
            else:
                fused.cfg_euler_step_(v, None, lat, 1.0, self.scheduler.dt(i), False, lat_lp)
        if (sp.output_type or self.od_config.output_type) == "latent":
            return DiffusionOutput(output=lat)
        return DiffusionOutput(output=(self.vae_decode or self.vae.decode)(unpack_latents(lat, h, w)))


class QwenImageEditPlusPipeline(QwenImageEditPipeline):
    max_condition_images = 3
    vl_image_area = 384 * 384
    picture_prefix = True


class QwenImageLayeredPipeline(QwenImageEditPipeline):
    """Layer decomposition: generates ``sampling_params.layers`` images of one scene as one batch
    conditioned on the same input image."""

    @torch.no_grad()
    def forward(self, req) -> DiffusionOutput:
        layers = max(1, int(req.sampling_params.layers))
        outs = []
        base_seed = req.sampling_params.seed or 0
        for k in range(layers):
            sp = req.sampling_params.clone() if req.sampling_params.generator is None else req.sampling_params
            sp.seed = base_seed + k
            sp.generator = None
            r = type(req)(req.prompts, sp, req.request_ids)
            outs.append(QwenImageEditPipeline.forward(self, r).output)
        return DiffusionOutput(output=torch.cat(outs, dim=0))
