"""TeaCache: skip the whole block stack when the timestep-modulated input barely moved.

Semantics of the reference hook (vllm_omni/diffusion/cache/teacache/hook.py:87-232,
config.py): metric = rel-L1 distance between this step's and the previous step's modulated
input of block 0, rescaled by a model-specific 4th-order polynomial and accumulated; while the
accumulator stays below ``rel_l1_thresh`` the blocks are skipped and the cached residual
(output - input of the stack) is re-applied; first and last step always compute.

The metric, polynomial, accumulation and decision run in one device kernel pair
(csrc/elementwise.cu: omni_rel_l1); the host reads back one 4-byte flag per step to decide
whether to launch the blocks (the reference reduces with several eager kernels and
synchronises on ``.cpu().item()``).
"""
from __future__ import annotations

import torch

from ...ops import fused
from .base import BlockStack, CacheBackend

MODEL_COEFFICIENTS = {
    "FluxTransformer2DModel": [4.98651651e02, -2.83781631e02, 5.58554382e01, -3.82021401e00, 2.64230861e-01],
    "QwenImageTransformer2DModel": [-4.5e02, 2.8e02, -4.5e01, 3.2e00, -2.0e-02],
    "ZImageTransformer2DModel": [-4.5e02, 2.8e02, -4.5e01, 3.2e00, -2.0e-02],
    "Bagel": [1.33313129e06, -1.68644226e05, 7.95050740e03, -1.63747873e02, 1.26352397e00],
}


class TeaCacheBackend(CacheBackend):
    name = "tea_cache"
    _branch_attrs = ("step", "state", "prev_mod", "residual")

    def __init__(self, config):
        super().__init__(config)
        self.thresh = float(getattr(config, "rel_l1_thresh", 0.2))
        self.coefficients = getattr(config, "coefficients", None)
        self.num_steps = 0
        self.step = 0
        self.state = None
        self.prev_mod = None
        self.residual = None

    def enable(self, pipeline):
        super().enable(pipeline)
        if self.coefficients is None:
            name = type(self.transformer).__name__
            name = {"BagelMoT": "Bagel"}.get(name, name)
            self.coefficients = MODEL_COEFFICIENTS.get(name, MODEL_COEFFICIENTS["QwenImageTransformer2DModel"])
        if len(self.coefficients) != 5:
            raise ValueError(f"coefficients must contain exactly 5 elements, got {len(self.coefficients)}")

    def refresh(self, pipeline, num_inference_steps=None):
        super().refresh(pipeline, num_inference_steps)
        self.num_steps = int(num_inference_steps or 0)
        self.step = 0
        self.state = None
        self.prev_mod = None
        self.residual = None
        self._remember_fresh_state()

    def on_stack(self, stack: BlockStack) -> tuple:
        self._switch_branch(stack.branch)
        cur = stack.probe.contiguous()
        states, L = stack.states, stack.num_blocks
        if self.state is None:
            self.state = fused.RelL1State(cur.device, self.coefficients, self.thresh)
        first_or_last = self.step == 0 or (self.num_steps and self.step == self.num_steps - 1)
        skip = False
        if self.prev_mod is not None and self.residual is not None and self.prev_mod.shape == cur.shape:
            fused.rel_l1_update(cur, self.prev_mod, self.state, force_compute=bool(first_or_last))
            skip = bool(self.state.state[2].item() > 0.5)       # the one host read-back of this step
        self.prev_mod = cur
        self.step += 1
        self.stats["steps"] += 1
        if skip:
            self.stats["skipped_steps"] += 1
            self.stats["skipped_blocks"] += L
            return tuple(s.add_(r) for s, r in zip(states, self.residual))
        before = tuple(s.clone() for s in states)
        out = stack.run(states, 0, L)
        self.residual = tuple(o - b for o, b in zip(out, before))
        self.stats["computed_blocks"] += L
        return out

    def _hook(self, model, run_blocks, img, txt, mods, cos, sin, kv_lens, ws, temb):
        """Qwen-Image entry: the probe is the image stream under block 0's modulation; blocks run in place."""
        D = model.cfg.inner_dim
        m0 = mods[:, 0, 0]
        cur = fused.norm_modulate(img, shift=m0[:, 0:D], scale=m0[:, D:2 * D], eps=model.cfg.eps)

        def run(states, a, b):
            run_blocks(img, txt, mods, cos, sin, kv_lens, ws, a, b)
            return (img, txt)
        return self.on_stack(BlockStack(model.cfg.num_layers, (img, txt), cur, run))
