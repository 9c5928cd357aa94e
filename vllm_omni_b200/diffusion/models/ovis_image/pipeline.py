"""Ovis-Image pipeline (vllm_omni/diffusion/models/ovis_image/): FLUX-family MMDiT with 6
double-stream and 27 single-stream blocks with gated MLPs and an Ovis text encoder."""
from __future__ import annotations

from ..flux.pipeline import FluxPipeline
from .transformer import OvisImageTransformer2DModel, OvisTransformerConfig


class OvisImagePipeline(FluxPipeline):
    transformer_cls, config_cls = OvisImageTransformer2DModel, OvisTransformerConfig
    default_guidance = 5.0
    true_cfg = True                             # guidance against the negative prompt
