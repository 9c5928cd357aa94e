"""LoRA adapters for diffusion transformers (vllm_omni/diffusion/lora/manager.py,
lora/layers/base_linear.py, vllm_omni/lora/{request,utils}.py).

Adapters are PEFT directories (``adapter_config.json`` + ``adapter_model.safetensors``).
Checkpoint module names go through the transformer's ``checkpoint_name_map`` so that LoRA
weights trained against the unfused diffusers modules (``to_q`` / ``to_k`` / ``to_v``) land
on the fused ``to_qkv`` rows they belong to (packed-module mapping).  Loaded adapters are kept
on the CPU in an LRU cache (``max_cached``), can be pinned, and are activated per request:
``y += scale * (x A^T) B^T`` with A, B on the GPU.
"""
from __future__ import annotations

import hashlib
import json
import os
from collections import OrderedDict

import torch

from ...inputs.data import LoRARequest
from ...logger import init_logger
from ..layers.linear import FusedLinear

logger = init_logger(__name__)


def stable_lora_int_id(name: str, path: str) -> int:
    return (int.from_bytes(hashlib.sha256(f"{name}:{path}".encode()).digest()[:4], "little") & 0x7FFFFFFF) or 1


class LoRAAdapter:
    def __init__(self, name: str, lora_id: int, rank: int, alpha: float, weights: dict):
        self.name, self.id, self.rank, self.alpha = name, lora_id, rank, alpha
        self.weights = weights          # module path -> list of (row_slice | None, A [r, in], B [rows, r])
        self.pinned = False

    @property
    def scaling(self) -> float:
        return self.alpha / max(self.rank, 1)


class DiffusionLoRAManager:
    def __init__(self, pipeline, max_cached: int | None = None):
        self.pipeline = pipeline
        self.transformer = pipeline.transformer
        self.max_cached = max_cached or 8
        self.adapters: "OrderedDict[int, LoRAAdapter]" = OrderedDict()
        self.active: list[tuple[int, float]] = []
        self._modules = {n: m for n, m in self.transformer.named_modules() if isinstance(m, FusedLinear)}
        # diffusers module path ("transformer_blocks.0.attn.to_q") -> (our module path, row slice)
        self._name_map = {}
        if hasattr(self.transformer, "checkpoint_name_map"):
            for ck, (pn, sl) in self.transformer.checkpoint_name_map().items():
                if ck.endswith(".weight") and pn.endswith(".weight"):
                    self._name_map[ck[:-len(".weight")]] = (pn[:-len(".weight")], sl)

    # ------------------------------------------------------------------ loading
    def load_adapter(self, name: str, path: str) -> LoRAAdapter:
        with open(os.path.join(path, "adapter_config.json")) as f:
            cfg = json.load(f)
        rank, alpha = int(cfg.get("r", 8)), float(cfg.get("lora_alpha", cfg.get("r", 8)))
        from ...utils.safetensors_reader import open_safetensors
        st = open_safetensors(os.path.join(path, "adapter_model.safetensors"))
        pairs: dict[str, dict] = {}
        for key in st.keys():
            k = key
            for pre in ("base_model.model.", "transformer.", "model."):
                if k.startswith(pre):
                    k = k[len(pre):]
            for tag, which in ((".lora_A.weight", "A"), (".lora_B.weight", "B"), (".lora_A.default.weight", "A"),
                               (".lora_B.default.weight", "B"), (".lora_down.weight", "A"), (".lora_up.weight", "B")):
                if k.endswith(tag):
                    pairs.setdefault(k[:-len(tag)], {})[which] = st.get_tensor(key).clone()
        weights: dict[str, list] = {}
        skipped = 0
        for mod, ab in pairs.items():
            if "A" not in ab or "B" not in ab:
                continue
            tgt = self._name_map.get(mod)
            if tgt is None and mod in self._modules:
                tgt = (mod, None)
            if tgt is None or tgt[0] not in self._modules:
                skipped += 1
                continue
            weights.setdefault(tgt[0], []).append((tgt[1], ab["A"], ab["B"]))
        if skipped:
            logger.warning("LoRA %s: %d modules have no counterpart in this transformer", name, skipped)
        if not weights:
            raise ValueError(f"LoRA adapter at {path} matches no module of {type(self.transformer).__name__}")
        return LoRAAdapter(name, stable_lora_int_id(name, path), rank, alpha, weights)

    def add_adapter_from_path(self, name: str, path: str, scale: float = 1.0) -> int:
        ad = self.load_adapter(name, path)
        self._insert(ad)
        return ad.id

    def add_adapter_from_request(self, req: LoRARequest, scale: float = 1.0) -> bool:
        if req.lora_int_id in self.adapters:
            self.adapters.move_to_end(req.lora_int_id)
            return True
        ad = self.load_adapter(req.lora_name, req.lora_path)
        ad.id = req.lora_int_id
        self._insert(ad)
        return True

    def _insert(self, ad: LoRAAdapter) -> None:
        self.adapters[ad.id] = ad
        self.adapters.move_to_end(ad.id)
        while len(self.adapters) > self.max_cached:
            victim = next((i for i, a in self.adapters.items() if not a.pinned and i not in [x for x, _ in self.active]),
                          None)
            if victim is None:
                break
            self.adapters.pop(victim)

    def remove_adapter(self, lora_id: int) -> bool:
        if lora_id in [i for i, _ in self.active]:
            self.set_active([(i, s) for i, s in self.active if i != lora_id])
        return self.adapters.pop(lora_id, None) is not None

    def list_adapters(self) -> list[int]:
        return list(self.adapters)

    def pin_adapter(self, lora_id: int) -> bool:
        if lora_id not in self.adapters:
            return False
        self.adapters[lora_id].pinned = True
        return True

    # ------------------------------------------------------------------ activation
    def set_active(self, adapters) -> None:
        """adapters: list of names / ids or (id, scale) pairs; empty list disables LoRA."""
        resolved = []
        for a in adapters:
            lid, scale = a if isinstance(a, tuple) else (a, 1.0)
            if isinstance(lid, str):
                lid = next((i for i, ad in self.adapters.items() if ad.name == lid), None)
            if lid is None or lid not in self.adapters:
                raise KeyError(f"LoRA adapter {a!r} is not loaded")
            resolved.append((lid, float(scale)))
        for m in self._modules.values():
            m.lora = None
        for lid, scale in resolved:
            ad = self.adapters[lid]
            for path, parts in ad.weights.items():
                m = self._modules[path]
                dev, dt = m.weight.device, m.weight.dtype
                for sl, A, B in parts:
                    if sl is not None:          # packed module: pad B to the fused width
                        Bf = torch.zeros(m.out_features, B.shape[1], dtype=dt, device=dev)
                        Bf[sl[0]:sl[1]] = B.to(dev, dt)
                    else:
                        Bf = B.to(dev, dt)
                    r = A.shape[0]
                    rp = (r + 7) // 8 * 8       # the GEMM wants K and N in multiples of 8
                    Ap = torch.zeros(rp, A.shape[1], dtype=dt, device=dev)
                    Ap[:r] = A.to(dev, dt)
                    Bp = torch.zeros(Bf.shape[0], rp, dtype=dt, device=dev)
                    Bp[:, :r] = Bf
                    m.lora = (m.lora or []) + [(Ap, Bp, ad.scaling * scale)]
        self.active = resolved
        tr = getattr(self.pipeline, "transformer", None) if hasattr(self, "pipeline") else None
        if tr is not None:
            tr._lora_active = bool(resolved)       # captured forwards bake the linears in: run eagerly with adapters

    def activate_request(self, req: LoRARequest, scale: float = 1.0) -> None:
        self.add_adapter_from_request(req, scale)
        want = [(req.lora_int_id, float(scale) * float(getattr(req, "scale", 1.0)))]
        if want != self.active:
            self.set_active(want)
