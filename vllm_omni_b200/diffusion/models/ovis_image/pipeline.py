"""Ovis-Image pipeline (vllm_omni/diffusion/models/ovis_image/): FLUX-family MMDiT with 6
double-stream and 27 single-stream blocks and an Ovis text encoder."""
from __future__ import annotations

from dataclasses import dataclass

from ..flux.pipeline import FluxPipeline
from ..flux.transformer import FluxTransformer2DModel, FluxTransformerConfig


@dataclass
class OvisTransformerConfig(FluxTransformerConfig):
    num_layers: int = 6
    num_single_layers: int = 27
    joint_attention_dim: int = 2048
    guidance_embeds: bool = False


class OvisImagePipeline(FluxPipeline):
    transformer_cls, config_cls = FluxTransformer2DModel, OvisTransformerConfig
    default_guidance = 5.0
