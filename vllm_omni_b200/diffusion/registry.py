"""Pipeline registry: ``model_index.json`` ``_class_name`` -> pipeline class, plus the pre-
and post-processing functions the engine runs around a pipeline call
(vllm_omni/diffusion/registry.py:122-293).
"""
from __future__ import annotations

import importlib
from typing import Callable

import torch

from .data import OmniDiffusionConfig

# class name -> (module under vllm_omni_b200.diffusion.models, class)
_DIFFUSION_MODELS: dict[str, tuple[str, str]] = {
    "QwenImagePipeline": ("qwen_image.pipeline", "QwenImagePipeline"),
    "QwenImageEditPipeline": ("qwen_image.pipeline_edit", "QwenImageEditPipeline"),
    "QwenImageEditPlusPipeline": ("qwen_image.pipeline_edit", "QwenImageEditPlusPipeline"),
    "QwenImageLayeredPipeline": ("qwen_image.pipeline_edit", "QwenImageLayeredPipeline"),
    "TinyMMDiTPipeline": ("tiny_mmdit.pipeline", "TinyMMDiTPipeline"),
    "WanPipeline": ("wan.pipeline", "WanPipeline"),
    "WanImageToVideoPipeline": ("wan.pipeline", "WanImageToVideoPipeline"),
    "Wan22TI2VPipeline": ("wan.pipeline", "WanTI2VPipeline"),
    "FluxPipeline": ("flux.pipeline", "FluxPipeline"),
    "Flux2KleinPipeline": ("flux2.pipeline", "Flux2KleinPipeline"),
    "ZImagePipeline": ("z_image.pipeline", "ZImagePipeline"),
    "StableDiffusion3Pipeline": ("sd3.pipeline", "StableDiffusion3Pipeline"),
    "LongCatImagePipeline": ("longcat_image.pipeline", "LongCatImagePipeline"),
    "LongCatImageEditPipeline": ("longcat_image.pipeline", "LongCatImageEditPipeline"),
    "OvisImagePipeline": ("ovis_image.pipeline", "OvisImagePipeline"),
    "GlmImagePipeline": ("glm_image.pipeline", "GlmImagePipeline"),
    "BagelPipeline": ("bagel.pipeline", "BagelPipeline"),
    "HunyuanImage3Pipeline": ("hunyuan_image_3.pipeline", "HunyuanImage3Pipeline"),
    "StableAudioPipeline": ("stable_audio.pipeline", "StableAudioPipeline"),
}

_VAE_PATCH_PARALLEL_ALLOWLIST = {"ZImagePipeline", "QwenImagePipeline", "FluxPipeline", "TinyMMDiTPipeline"}
_AUDIO_OUTPUT = {"StableAudioPipeline"}
_VIDEO_OUTPUT = {"WanPipeline", "WanImageToVideoPipeline", "Wan22TI2VPipeline"}


def register_diffusion_model(class_name: str, module: str, cls: str) -> None:
    """Plugin hook: ``module`` may be a fully-qualified module path."""
    _DIFFUSION_MODELS[class_name] = (module, cls)


def supported_models() -> list[str]:
    return sorted(_DIFFUSION_MODELS)


def supports_audio_output(class_name: str | None) -> bool:
    return class_name in _AUDIO_OUTPUT


def supports_video_output(class_name: str | None) -> bool:
    return class_name in _VIDEO_OUTPUT


def resolve_pipeline_class(class_name: str):
    if class_name not in _DIFFUSION_MODELS:
        raise ValueError(f"Model class {class_name} not found in diffusion model registry: {supported_models()}")
    mod, cls = _DIFFUSION_MODELS[class_name]
    full = mod if mod.startswith("vllm_omni_b200.") or "." in mod and not mod.split(".")[0] in _local_pkgs() \
        else f"vllm_omni_b200.diffusion.models.{mod}"
    return getattr(importlib.import_module(full), cls)


def _local_pkgs():
    return {m.split(".")[0] for m, _ in _DIFFUSION_MODELS.values()}


def initialize_model(od_config: OmniDiffusionConfig, device=None):
    """Instantiate the pipeline, attach sequence-parallel plans and VAE patch parallelism."""
    extra = {}
    if od_config.diffusion_load_format == "custom_pipeline":
        # a user class behind the engine (vllm_omni/diffusion/model_loader/diffusers_loader.py:217-226,
        # worker/diffusion_worker.py:291-311): ``custom_pipeline_args["pipeline_class"]`` is its qualified
        # name, the other keys are keyword arguments of its constructor
        args = dict(od_config.custom_pipeline_args or {})
        name = args.pop("pipeline_class", None)
        if not name:
            raise ValueError("diffusion_load_format='custom_pipeline' needs custom_pipeline_args['pipeline_class']")
        mod, _, attr = name.rpartition(".")
        cls, extra = getattr(importlib.import_module(mod), attr), args
    else:
        cls = resolve_pipeline_class(od_config.model_class_name)
    pipe = cls(od_config, device=device, **extra)
    pc = od_config.parallel_config
    if pc.sequence_parallel_size > 1 or pc.cfg_parallel_size > 1 or pc.tensor_parallel_size > 1:
        from ..parallel.apply import apply_parallelism
        apply_parallelism(pipe, od_config)
    if pc.vae_patch_parallel_size > 1 and od_config.model_class_name in _VAE_PATCH_PARALLEL_ALLOWLIST:
        from ..parallel.vae_patch_parallel import VaePatchParallelism
        VaePatchParallelism(pipe, pc.vae_patch_parallel_size).install()
    return pipe


# ------------------------------------------------------------------ pre / post processing
def tensor_to_pil(images: torch.Tensor) -> list:
    """[B, 3, H, W] in [-1, 1] -> list of PIL images."""
    from PIL import Image
    x = ((images.float().clamp(-1, 1) + 1) * 127.5).round().to(torch.uint8)
    x = x.permute(0, 2, 3, 1).cpu().numpy()
    return [Image.fromarray(a) for a in x]


def get_post_process_func(od_config: OmniDiffusionConfig) -> Callable | None:
    name = od_config.model_class_name
    if supports_audio_output(name):
        return lambda audio: [a.float().cpu() for a in audio]
    if supports_video_output(name):
        def video_post(frames: torch.Tensor):
            # [B, 3, T, H, W] in [-1, 1] -> list of uint8 arrays [T, H, W, 3]
            x = ((frames.float().clamp(-1, 1) + 1) * 127.5).round().to(torch.uint8)
            return [v.permute(1, 2, 3, 0).cpu().numpy() for v in x]
        return video_post

    def image_post(images):
        if od_config.output_type in ("pt", "latent") or not isinstance(images, torch.Tensor) or images.dim() != 4:
            return images if isinstance(images, list) else list(images)
        return tensor_to_pil(images)
    return image_post


def get_pre_process_func(od_config: OmniDiffusionConfig) -> Callable | None:
    """Image-conditioned pipelines turn PIL / array inputs into [-1, 1] tensors here."""
    if od_config.model_class_name not in {"QwenImageEditPipeline", "QwenImageEditPlusPipeline",
                                          "QwenImageLayeredPipeline", "WanImageToVideoPipeline",
                                          "Wan22TI2VPipeline", "LongCatImageEditPipeline"}:
        return None

    def pre(req):
        import numpy as np
        for p in req.prompts:
            if isinstance(p, str):
                continue
            mm = p.get("multi_modal_data") or {}
            img = mm.get("image")
            if img is None:
                continue
            imgs = img if isinstance(img, (list, tuple)) else [img]
            out = []
            for im in imgs:
                if isinstance(im, torch.Tensor):
                    out.append(im)
                    continue
                a = np.asarray(im.convert("RGB") if hasattr(im, "convert") else im, dtype=np.float32) / 127.5 - 1.0
                out.append(torch.from_numpy(a).permute(2, 0, 1))
            mm["image_tensor"] = out
        return req
    return pre
