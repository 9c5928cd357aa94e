"""Weight offloading (vllm_omni/diffusion/offloader/: layerwise_backend.py, sequential_backend.py).

``LayerWiseOffloadBackend``: transformer blocks live in pinned host memory as one flat buffer
per block; a copy stream prefetches block i+1 while block i computes, and a block's GPU copy
is dropped after use, so resident weights are two blocks instead of all of them.
``ModelLevelOffloadBackend``: whole components (text encoder / transformer / VAE) are swapped
between host and device around their use, never two large ones at once.
"""
from __future__ import annotations

import torch
from torch import nn


def get_offload_backend(od_config, device):
    if device.type != "cuda":
        return None
    if od_config.enable_layerwise_offload:
        return LayerWiseOffloadBackend(device, od_config.pin_cpu_memory)
    if od_config.enable_cpu_offload:
        return ModelLevelOffloadBackend(device, od_config.pin_cpu_memory)
    return None


class LayerWiseOffloadBackend:
    blocks_attr_candidates = ("blocks", "transformer_blocks", "layers")

    def __init__(self, device, pin: bool = True):
        self.device, self.pin = device, pin
        self.copy_stream = None
        self.host: list[torch.Tensor] = []
        self.layout: list[list] = []
        self.events: dict[int, torch.cuda.Event] = {}
        self.resident: dict[int, torch.Tensor] = {}

    def _blocks(self, model) -> nn.ModuleList:
        for n in self.blocks_attr_candidates:
            b = getattr(model, n, None)
            if isinstance(b, nn.ModuleList) and len(b):
                return b
        raise ValueError(f"{type(model).__name__} has no block list to offload")

    def enable(self, pipeline) -> None:
        tr = pipeline.transformer
        self.model = tr
        self.blocks = self._blocks(tr)
        self.copy_stream = torch.cuda.Stream(self.device)
        for blk in self.blocks:
            params = [p for p in blk.parameters()]
            total = sum(p.numel() * p.element_size() for p in params)
            flat = torch.empty(total, dtype=torch.uint8, pin_memory=self.pin)
            lay, off = [], 0
            for p in params:
                n = p.numel() * p.element_size()
                flat[off:off + n].copy_(p.data.detach().contiguous().view(torch.uint8).reshape(-1).cpu())
                lay.append((p, off, n, p.shape, p.dtype))
                p.data = torch.empty(0, dtype=p.dtype, device=self.device)
                off += n
            self.host.append(flat)
            self.layout.append(lay)
        torch.cuda.empty_cache()
        orig = tr._run_blocks

        def run_blocks(img, txt, mods, cos, sin, kv_lens, ws, start=0, end=None):
            end = tr.cfg.num_layers if end is None else end
            self.prefetch(start)
            for i in range(start, end):
                if i + 1 < end:
                    self.prefetch(i + 1)
                self.wait(i)
                tr.block_forward(i, img, txt, mods, cos, sin, kv_lens, ws)
                self.release(i)
            return img, txt
        tr._run_blocks = run_blocks
        self._orig = orig

    def prefetch(self, i: int) -> None:
        if i in self.resident:
            return
        with torch.cuda.stream(self.copy_stream):
            dev = self.host[i].to(self.device, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.copy_stream)
        self.resident[i] = dev
        self.events[i] = ev

    def wait(self, i: int) -> None:
        torch.cuda.current_stream().wait_event(self.events[i])
        dev = self.resident[i]
        for p, off, n, shape, dtype in self.layout[i]:
            p.data = dev[off:off + n].view(dtype).view(shape)

    def release(self, i: int) -> None:
        dev = self.resident.pop(i)
        dev.record_stream(torch.cuda.current_stream())
        for p, *_ in self.layout[i]:
            p.data = torch.empty(0, dtype=p.dtype, device=self.device)
        self.events.pop(i, None)


class ModelLevelOffloadBackend:
    def __init__(self, device, pin: bool = True):
        self.device, self.pin = device, pin
        self.components: dict[str, nn.Module] = {}
        self.on_device: str | None = None

    def enable(self, pipeline) -> None:
        for name in ("text_encoder", "transformer", "vae"):
            m = getattr(pipeline, name, None)
            if isinstance(m, nn.Module):
                self.components[name] = m
                m.to("cpu")
        torch.cuda.empty_cache()
        self.pipeline = pipeline

    def use(self, name: str) -> nn.Module:
        """Bring ``name`` to the GPU, evicting whichever large component is there."""
        if self.on_device and self.on_device != name:
            self.components[self.on_device].to("cpu")
            torch.cuda.empty_cache()
        self.components[name].to(self.device)
        self.on_device = name
        return self.components[name]
