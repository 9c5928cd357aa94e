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


def safetensors_weights_iterator(files: list[str], prefix: str = "", num_threads: int = 8) -> Iterator:
    """Yields (prefix + name, tensor).  Each shard is read by the C++ reader: its tensors are copied
    out of the mapping by ``num_threads`` workers into one host buffer, which overlaps the page
    faults of a cold file; the next shard is read while the current one is consumed.
    ``OMNI_LOADER=mmap`` yields zero-copy views of the mapping instead (one page fault at a time)."""
    from ..utils.safetensors_reader import NativeSafetensorsFile, open_safetensors

    def load(path):
        if os.environ.get("OMNI_LOADER", "native") != "mmap":
            try:
                f = NativeSafetensorsFile(path, threads=num_threads)
                try:
                    return f.read(pin=False)
                finally:
                    f.close()
            except (OSError, RuntimeError) as e:          # library not buildable here: fall back
                logger.warning("native safetensors reader unavailable (%s); using the mmap reader", e)
        st = open_safetensors(path)
        return {name: st.get_tensor(name) for name in st.keys()}

    with ThreadPoolExecutor(max_workers=2) as ex:
        for tensors in ex.map(load, files):
            for name, t in tensors.items():
                yield prefix + name, t


class DiffusersPipelineLoader:
    COMPONENTS = ("transformer", "transformer_2", "vae", "text_encoder", "text_encoder_2", "text_encoder_3",
                  "projection_model")

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
