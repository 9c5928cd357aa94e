"""GLM-Image pipeline (vllm_omni/diffusion/models/glm_image/): a double-stream MMDiT decoder that
runs true CFG; its reference implementation carries an inline copy of CFG-parallel
(pipeline_glm_image.py:713-724) — here it uses the shared ``CFGExchange`` like every pipeline."""
from __future__ import annotations

from dataclasses import dataclass

from ..qwen_image.pipeline import QwenImagePipeline
from ..qwen_image.transformer import QwenImageTransformerConfig


@dataclass
class GlmImageTransformerConfig(QwenImageTransformerConfig):
    num_layers: int = 30
    attention_head_dim: int = 128
    num_attention_heads: int = 32
    joint_attention_dim: int = 4096


class GlmImagePipeline(QwenImagePipeline):
    def __init__(self, od_config=None, transformer_config=None, vae_config=None, device=None, **kw):
        tc = transformer_config or GlmImageTransformerConfig.from_dict(od_config.tf_model_config.to_dict() if od_config else {})
        super().__init__(od_config, tc, vae_config, device)
