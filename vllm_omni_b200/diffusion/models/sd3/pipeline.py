"""Stable Diffusion 3 pipeline (vllm_omni/diffusion/models/sd3/): joint-attention MMDiT blocks
(the double-stream block of the FLUX family without single-stream blocks), pooled CLIP vector +
timestep conditioning, classifier-free guidance with cond/uncond batched."""
from __future__ import annotations

from dataclasses import dataclass

from ..flux.pipeline import FluxPipeline
from ..flux.transformer import FluxTransformer2DModel, FluxTransformerConfig


@dataclass
class SD3TransformerConfig(FluxTransformerConfig):
    num_layers: int = 24
    num_single_layers: int = 0
    attention_head_dim: int = 64
    num_attention_heads: int = 24
    joint_attention_dim: int = 4096
    pooled_projection_dim: int = 2048
    guidance_embeds: bool = False
    axes_dims_rope: tuple = (16, 24, 24)


class SD3Transformer2DModel(FluxTransformer2DModel):
    pass


class StableDiffusion3Pipeline(FluxPipeline):
    transformer_cls, config_cls = SD3Transformer2DModel, SD3TransformerConfig
    default_guidance = 7.0
    max_text_len = 333
