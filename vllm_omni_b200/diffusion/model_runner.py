"""Runs a pipeline on one rank: load, attach acceleration (cache, offload, LoRA), execute
(vllm_omni/diffusion/worker/diffusion_model_runner.py:70-202)."""
from __future__ import annotations

import time

import torch

from ..utils.safetensors_reader import NvtxRange

from ..logger import init_logger
from .data import DiffusionOutput, OmniDiffusionConfig
from .forward_context import set_forward_context
from .loader import DiffusersPipelineLoader
from .request import OmniDiffusionRequest

logger = init_logger(__name__)


class DiffusionModelRunner:
    def __init__(self, od_config: OmniDiffusionConfig, device: torch.device):
        self.od_config = od_config
        self.device = device
        self.pipeline = None
        self.cache_backend = None
        self.offload_backend = None
        self.kv_transfer_manager = None

    def load_model(self):
        t0 = time.perf_counter()
        self.pipeline = DiffusersPipelineLoader(self.od_config).load_model(self.device)
        cfg = self.od_config
        if cfg.enable_cpu_offload or cfg.enable_layerwise_offload:
            from .offloader import get_offload_backend
            self.offload_backend = get_offload_backend(cfg, self.device)
            if self.offload_backend is not None:
                self.offload_backend.enable(self.pipeline)
        if cfg.cache_backend not in (None, "none"):
            from .cache.selector import get_cache_backend
            self.cache_backend = get_cache_backend(cfg.cache_backend, cfg.cache_config)
            self.cache_backend.enable(self.pipeline)
        if not (cfg.enable_cpu_offload or cfg.enable_layerwise_offload):
            from .graphed import maybe_graph_transformer
            if maybe_graph_transformer(self.pipeline, cfg):
                logger.info("denoiser forward will be replayed from CUDA graphs")
        if cfg.omni_kv_config:
            from ..connectors.kv_transfer_manager import OmniKVTransferManager
            self.kv_transfer_manager = OmniKVTransferManager.from_config(cfg.omni_kv_config)
        logger.info("model loaded in %.1f s", time.perf_counter() - t0)
        return self.pipeline

    @torch.no_grad()
    def execute_model(self, req: OmniDiffusionRequest) -> DiffusionOutput:
        assert self.pipeline is not None, "load_model() first"
        sp = req.sampling_params
        if self.kv_transfer_manager is not None and sp.need_kv_receive and sp.past_key_values is None:
            self.kv_transfer_manager.receive_kv_cache(req, target_device=self.device)
        if sp.generator is None and sp.seed is not None:
            sp.generator = torch.Generator(device="cpu").manual_seed(int(sp.seed))
        if self.cache_backend is not None:
            self.cache_backend.refresh(self.pipeline, sp.num_inference_steps)
        with set_forward_context(od_config=self.od_config, num_steps=sp.num_inference_steps):
            with torch.profiler.record_function("pipeline_forward"), NvtxRange("pipeline_forward"):
                try:
                    return self.pipeline.forward(req)
                except Exception as e:   # surfaced to the engine as a typed error result
                    logger.exception("pipeline forward failed")
                    import traceback
                    return DiffusionOutput(error=f"{type(e).__name__}: {e}\n{traceback.format_exc()}")
