"""LongCat-Image pipelines (vllm_omni/diffusion/models/longcat_image/): FLUX-family MMDiT
(19 double + 38 single blocks at width 3072) with a Qwen2.5-VL text encoder; the edit variant
appends the VAE latents of the input image to the image sequence."""
from __future__ import annotations

import torch

from ..flux.pipeline import FluxPipeline
from .transformer import LongCatImageTransformer2DModel, LongCatTransformerConfig


class LongCatImagePipeline(FluxPipeline):
    transformer_cls, config_cls = LongCatImageTransformer2DModel, LongCatTransformerConfig
    default_guidance = 4.5
    true_cfg, cfg_renorm_clamp = True, True     # guidance against the negative prompt, guided velocity clamped per token


class LongCatImageEditPipeline(LongCatImagePipeline):
    """Image editing (vllm_omni/diffusion/models/longcat_image/pipeline_longcat_image_edit.py:417-485,
    640-690): the input image is encoded by the VAE, packed like the noise latents and appended to
    the image sequence as a second frame whose rotary position carries modality id 2 (the noise rows
    are modality 1); the network sees [noise rows | condition rows | text], only the noise rows'
    velocity is kept and stepped.  The image arrives as ``multi_modal_data['image_tensor']``
    ([-1, 1] tensors, see ``registry.get_pre_process_func``), or as ready latents in
    ``multi_modal_data['image_latents']``."""
    needs_vae_encoder = True

    def condition_latents(self, req, B, h, w):
        from ..qwen_image.pipeline import pack_latents
        lats = []
        for p in req.prompts:
            mm = (p.get("multi_modal_data") or {}) if isinstance(p, dict) else {}
            if mm.get("image_latents") is not None:
                z = mm["image_latents"].to(self.device_, torch.float32)
                z = z[None] if z.dim() == 3 else z
            else:
                imgs = mm.get("image_tensor") or []
                if not imgs:
                    raise ValueError("LongCatImageEditPipeline needs an input image (multi_modal_data['image'])")
                im = imgs[0].to(self.device_, torch.float32)[None]
                if im.shape[-2:] != (h * 8, w * 8):
                    im = torch.nn.functional.interpolate(im, size=(h * 8, w * 8), mode="bicubic", align_corners=False)
                z = self.vae.encode(im.clamp(-1, 1)).float()                   # posterior mode, scheduler space
            if z.shape[-2:] != (h, w):
                z = torch.nn.functional.interpolate(z, size=(h, w), mode="bilinear", align_corners=False)
            lats.append(pack_latents(z))
        cond = torch.cat(lats, dim=0)
        if cond.shape[0] != B:                       # several outputs per prompt
            cond = cond.repeat_interleave(B // cond.shape[0], dim=0)
        return cond
