"""Diffusion stage engines: ``OmniDiffusion`` (blocking) and ``AsyncOmniDiffusion``.

Model discovery follows the reference (vllm_omni/entrypoints/omni_diffusion.py,
async_omni_diffusion.py): ``model_index.json`` ``_class_name`` picks the pipeline and
``transformer/config.json`` becomes ``tf_model_config``.  A model argument that names a
registered pipeline class (e.g. ``"QwenImagePipeline"``) builds that architecture with
random weights (``load_format='dummy'``).
"""
from __future__ import annotations

import asyncio
import os
import uuid
from concurrent.futures import ThreadPoolExecutor
from dataclasses import fields
from typing import Any

from ..diffusion.data import DiffusionParallelConfig, OmniDiffusionConfig, TransformerConfig
from ..diffusion.engine import DiffusionEngine
from ..diffusion.loader import read_component_config, read_model_index
from ..diffusion.registry import _DIFFUSION_MODELS
from ..diffusion.request import OmniDiffusionRequest
from ..inputs.data import OmniDiffusionSamplingParams
from ..outputs import OmniRequestOutput


def build_diffusion_config(model: str | None = None, od_config: OmniDiffusionConfig | dict | None = None,
                           **kwargs) -> OmniDiffusionConfig:
    if isinstance(od_config, OmniDiffusionConfig):
        cfg = od_config
    else:
        kw = dict(od_config or {})
        kw.update(kwargs)
        if model is not None:
            kw["model"] = model
        pnames = {f.name for f in fields(DiffusionParallelConfig)}
        pc = kw.get("parallel_config")
        loose = {k: kw.pop(k) for k in list(kw) if k in pnames}
        if pc is None and loose:
            kw["parallel_config"] = DiffusionParallelConfig(**loose)
        names = {f.name for f in fields(OmniDiffusionConfig)}
        cfg = OmniDiffusionConfig(**{k: v for k, v in kw.items() if k in names})
    m = cfg.model
    if cfg.model_class_name is None:
        if m and os.path.isdir(m):
            idx = read_model_index(m)
            cfg.model_class_name = idx.get("_class_name")
            tc = read_component_config(m, "transformer")
            if tc and not cfg.tf_model_config.params:
                cfg.tf_model_config = TransformerConfig.from_dict(tc)
            vc = read_component_config(m, "vae")
            if vc and not cfg.vae_config:
                cfg.vae_config = vc
        elif m in _DIFFUSION_MODELS:
            cfg.model_class_name = m
            if cfg.diffusion_load_format != "custom_pipeline":
                cfg.diffusion_load_format = "dummy"
        elif m:
            guess = {"qwen-image": "QwenImagePipeline", "wan": "WanPipeline", "flux": "FluxPipeline",
                     "z-image": "ZImagePipeline", "stable-diffusion-3": "StableDiffusion3Pipeline",
                     "tiny-mmdit": "TinyMMDiTPipeline"}
            low = m.lower()
            for k, v in guess.items():
                if k in low:
                    cfg.model_class_name = v
                    if cfg.diffusion_load_format != "custom_pipeline":
                        cfg.diffusion_load_format = "dummy"
                    break
    if cfg.model_class_name is None:
        raise ValueError(f"cannot determine the pipeline class for model {m!r}; pass model_class_name")
    return cfg


class OmniDiffusion:
    def __init__(self, model: str | None = None, od_config=None, **kwargs):
        self.od_config = build_diffusion_config(model, od_config, **kwargs)
        self.engine = DiffusionEngine.make_engine(self.od_config)

    def generate(self, prompts, sampling_params: OmniDiffusionSamplingParams | None = None,
                 request_ids: list[str] | None = None) -> list[OmniRequestOutput]:
        if isinstance(prompts, (str, dict)):
            prompts = [prompts]
        sp = sampling_params or OmniDiffusionSamplingParams()
        ids = request_ids or [f"diff-{uuid.uuid4().hex[:8]}" for _ in prompts]
        return self.engine.step(OmniDiffusionRequest(list(prompts), sp, ids))

    def abort(self, request_ids):
        self.engine.abort(request_ids)

    def collective_rpc(self, method, timeout=None, args=(), kwargs=None):
        return self.engine.collective_rpc(method, timeout, args, kwargs)

    def start_profile(self, trace_dir=None):
        return self.engine.start_profile(trace_dir)

    def stop_profile(self):
        return self.engine.stop_profile()

    def close(self):
        self.engine.close()


class AsyncOmniDiffusion:
    """Async facade: the blocking ``engine.step`` runs on a single worker thread so the event
    loop stays responsive; LoRA management goes through ``collective_rpc``."""

    def __init__(self, model: str | None = None, od_config=None, **kwargs):
        self.od_config = build_diffusion_config(model, od_config, **kwargs)
        self.engine = DiffusionEngine.make_engine(self.od_config)
        self._pool = ThreadPoolExecutor(max_workers=1, thread_name_prefix="omni-diffusion")
        self._closed = False

    async def generate(self, prompt, sampling_params: OmniDiffusionSamplingParams | None = None,
                       request_id: str | None = None) -> OmniRequestOutput:
        rid = request_id or f"diff-{uuid.uuid4().hex[:8]}"
        sp = sampling_params or OmniDiffusionSamplingParams()
        req = OmniDiffusionRequest([prompt], sp, [rid])
        loop = asyncio.get_running_loop()
        outs = await loop.run_in_executor(self._pool, self.engine.step, req)
        if not outs:
            raise asyncio.CancelledError(f"request {rid} was aborted")
        return outs[0]

    async def abort(self, request_id):
        self.engine.abort(request_id)

    async def add_lora(self, lora_request, scale: float = 1.0):
        return await self._rpc("add_lora", (lora_request, scale))

    async def remove_lora(self, lora_id: int):
        return await self._rpc("remove_lora", (lora_id,))

    async def list_loras(self):
        return await self._rpc("list_loras")

    async def pin_lora(self, lora_id: int):
        return await self._rpc("pin_lora", (lora_id,))

    async def _rpc(self, method, args=()):
        loop = asyncio.get_running_loop()
        return await loop.run_in_executor(self._pool, lambda: self.engine.collective_rpc(method, args=args))

    async def check_health(self):
        if not self.engine.check_health():
            raise RuntimeError("diffusion workers are not healthy")

    def close(self):
        if not self._closed:
            self._closed = True
            self._pool.shutdown(wait=False)
            self.engine.close()

    shutdown = close
