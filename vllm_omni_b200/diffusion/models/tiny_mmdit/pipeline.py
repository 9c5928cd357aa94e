"""Tiny MMDiT text-to-image pipeline: the CPU / fp32 plumbing configuration.

Two double-stream blocks, hidden 128, 4 heads x 32, patch 2, 16-channel latents, 128-wide
text states, a small convolutional VAE decoder (8x up-sampling: 32x32 latents -> 256x256 RGB).
It is the same code as the Qwen-Image pipeline with a small configuration, so the Omni API,
stage configs, schedulers, CFG and caches can be exercised end to end without a GPU, and its
PyTorch path is the oracle the fused kernels are compared against.
"""
from __future__ import annotations

from ..qwen_image.pipeline import QwenImagePipeline
from ..qwen_image.transformer import QwenImageTransformerConfig
from ..vae.autoencoder_kl_qwenimage import QwenImageVAEConfig

TINY_TRANSFORMER = dict(num_layers=2, attention_head_dim=32, num_attention_heads=4, joint_attention_dim=128,
                        in_channels=64, out_channels=16, axes_dims_rope=(8, 12, 12))
TINY_VAE = dict(base_dim=8, z_dim=16, dim_mult=(1, 2, 4, 4), num_res_blocks=1,
                latents_mean=(0.0,) * 16, latents_std=(1.0,) * 16)
TINY_SCHEDULER = dict(num_train_timesteps=1000, shift=1.0, use_dynamic_shifting=False)


class TinyMMDiTPipeline(QwenImagePipeline):
    def __init__(self, od_config=None, transformer_config=None, vae_config=None, device=None, **kw):
        tc = dict(TINY_TRANSFORMER)
        if od_config is not None:
            tc.update({k: v for k, v in od_config.tf_model_config.to_dict().items() if k in tc})
        super().__init__(od_config, transformer_config or QwenImageTransformerConfig.from_dict(tc),
                         vae_config or QwenImageVAEConfig.from_dict(TINY_VAE), device=device,
                         scheduler_config=TINY_SCHEDULER)
        self.default_sample_size = 32
        self.text_encoder.max_len = 32
