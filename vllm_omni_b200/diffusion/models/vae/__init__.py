"""VAEs of the diffusion pipelines.  ``build_vae`` picks the class from the checkpoint's
``vae/config.json`` (``_class_name``), falling back to the family's usual autoencoder."""
from __future__ import annotations


def build_vae(vae_config: dict | None, family: str = "qwen", with_encoder: bool = False):
    """family: "qwen" (causal-3D Qwen-Image / Wan VAE in image mode) or "kl" (the 2-D AutoencoderKL of
    FLUX / SD3 / Z-Image checkpoints)."""
    vc = dict(vae_config or {})
    name = vc.get("_class_name")
    if name in ("AutoencoderKL", "AutoencoderKLFlux2") or (name is None and family == "kl"):
        from .autoencoder_kl import AutoencoderKL, AutoencoderKLConfig
        return AutoencoderKL(AutoencoderKLConfig.from_dict(vc), with_encoder=with_encoder)
    from .autoencoder_kl_qwenimage import AutoencoderKLQwenImage2d, QwenImageVAEConfig
    return AutoencoderKLQwenImage2d(QwenImageVAEConfig.from_dict(vc), with_encoder=with_encoder)
