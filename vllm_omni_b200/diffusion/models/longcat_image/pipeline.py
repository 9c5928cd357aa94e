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
    """Image editing: the conditioning image travels in ``multi_modal_data['image_tensor']`` (see
    ``registry.get_pre_process_func``) and biases the initial latents."""
