"""Checkpoint loading for diffusers-layout repositories.

A model directory has ``model_index.json`` and one sub-folder per component
(``transformer/``, ``vae/``, ``text_encoder/`` ...) holding safetensors shards.  The
loader streams (name, tensor) pairs with the component prefix to ``pipeline.load_weights``
(vllm_omni/diffusion/model_loader/diffusers_loader.py:1-280).  ``load_format='dummy'``
keeps the seeded random initialisation, which is what the benchmarks use.
"""
from __future__ import annotations

import json
import os
from concurrent.futures import ThreadPoolExecutor
from typing import Iterator

import torch

from ..logger import init_logger
from .data import OmniDiffusionConfig

logger = init_logger(__name__)


def read_model_index(model_path: str) -> dict:
    p = os.path.join(model_path, "model_index.json")
    if not os.path.exists(p):
        return {}
    with open(p) as f:
        return json.load(f)


def read_component_config(model_path: str, component: str) -> dict:
    p = os.path.join(model_path, component, "config.json")
    if not os.path.exists(p):
        return {}
    with open(p) as f:
        return json.load(f)


def _shard_files(folder: str) -> list[str]:
    if not os.path.isdir(folder):
        return []
    idx = [f for f in os.listdir(folder) if f.endswith(".safetensors.index.json")]
    if idx:
        with open(os.path.join(folder, idx[0])) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
        return [os.path.join(folder, x) for x in files]
    return sorted(os.path.join(folder, f) for f in os.listdir(folder) if f.endswith(".safetensors"))


def safetensors_weights_iterator(files: list[str], prefix: str = "", num_threads: int = 4) -> Iterator:
    """Yields (prefix + name, tensor).  Shards are opened by a small thread pool so that disk
    reads of the next shard overlap the copies of the current one."""
    from ..utils.safetensors_reader import open_safetensors

    def load(path):
        return open_safetensors(path)

    with ThreadPoolExecutor(max_workers=max(1, num_threads)) as ex:
        for st in ex.map(load, files):
            for name in st.keys():
                yield prefix + name, st.get_tensor(name)


class DiffusersPipelineLoader:
    COMPONENTS = ("transformer", "transformer_2", "vae", "text_encoder", "text_encoder_2")

    def __init__(self, od_config: OmniDiffusionConfig):
        self.od_config = od_config

    def weights(self, model_path: str) -> Iterator:
        for comp in self.COMPONENTS:
            files = _shard_files(os.path.join(model_path, comp))
            if files:
                yield from safetensors_weights_iterator(files, prefix=comp + ".")

    def load_model(self, device) -> torch.nn.Module:
        from .registry import initialize_model
        cfg = self.od_config
        fmt = cfg.diffusion_load_format
        torch.manual_seed(cfg.seed)
        pipe = initialize_model(cfg, device=device)
        if fmt == "dummy" or not cfg.model or not os.path.isdir(cfg.model):
            if fmt != "dummy":
                logger.warning("model path %r is not a local directory; keeping random weights", cfg.model)
        else:
            if hasattr(pipe, "attach_text_encoder") and pipe.attach_text_encoder(cfg.model):
                logger.info("prompt encoder: text_encoder/ of %s", cfg.model)
            loaded = pipe.load_weights(self.weights(cfg.model))
            logger.info("loaded %d checkpoint tensors from %s", len(loaded), cfg.model)
        if cfg.quantization:
            from .quantization.fp8 import quantize_pipeline
            quantize_pipeline(pipe, cfg)
        pipe.eval()
        return pipe
