"""DBCache + TaylorSeer + step-mask (the cache-dit feature set the reference enables through
the external ``cache_dit`` library, vllm_omni/diffusion/cache/cache_dit_backend.py:855-960).

Per step: always run the first ``Fn_compute_blocks``; compare their output's residual with the
one cached at the last fully computed step (rel-L1, on device).  Below
``residual_diff_threshold`` (and within the warm-up / continuous-step / total-step limits) the
middle blocks are skipped and their cached residual is applied — extrapolated by a
TaylorSeer polynomial of order ``taylorseer_order`` when enabled — then the last
``Bn_compute_blocks`` run.  ``scm_steps_mask_policy`` forces a fixed compute/cache pattern.
"""
from __future__ import annotations

import torch

from ...ops import fused
from .base import BlockStack, CacheBackend

SCM_POLICIES = {   # 1 = compute, 0 = may use the cache; the pattern repeats over the steps
    "slow": [1, 1, 0, 1, 1, 0], "medium": [1, 0, 1, 0], "fast": [1, 0, 0, 1, 0, 0], "ultra": [1, 0, 0, 0],
}


class TaylorSeer:
    """Finite-difference Taylor extrapolation of a cached tensor over steps."""

    def __init__(self, order: int = 1):
        self.order = max(0, int(order))
        self.derivs: list[torch.Tensor] = []
        self.last_step = None

    def update(self, y: torch.Tensor, step: int):
        new = [y]
        if self.last_step is not None and step > self.last_step:
            dt = float(step - self.last_step)
            for k in range(min(self.order, len(self.derivs))):
                new.append((new[k] - self.derivs[k]) / dt)
        self.derivs = new
        self.last_step = step

    def predict(self, step: int) -> torch.Tensor:
        dt = float(step - self.last_step)
        out = self.derivs[0].clone()
        f = 1.0
        for k in range(1, len(self.derivs)):
            f = f * dt / k
            out.add_(self.derivs[k], alpha=f)
        return out


class DBCacheBackend(CacheBackend):
    name = "cache_dit"
    _branch_attrs = ("step", "cached_steps", "cont", "prev_fn_res", "mid_res", "seers", "state")

    def __init__(self, config):
        super().__init__(config)
        g = lambda n, d: getattr(config, n, d)
        self.Fn, self.Bn = int(g("Fn_compute_blocks", 1)), int(g("Bn_compute_blocks", 0))
        self.warmup = int(g("max_warmup_steps", 4))
        self.max_cached = int(g("max_cached_steps", -1))
        self.max_cont = int(g("max_continuous_cached_steps", 3))
        self.thresh = float(g("residual_diff_threshold", 0.24))
        self.use_taylor = bool(g("enable_taylorseer", False))
        self.order = int(g("taylorseer_order", 1))
        self.scm = g("scm_steps_mask_policy", None)
        self.refresh(None)

    def refresh(self, pipeline, num_inference_steps=None):
        super().refresh(pipeline, num_inference_steps)
        self.step = 0
        self.cached_steps = 0
        self.cont = 0
        self.prev_fn_res = None
        self.mid_res = None
        self.seers: list = []
        self.state = None
        self._remember_fresh_state()

    def _may_cache(self) -> bool:
        if self.step < self.warmup:
            return False
        if self.max_cached >= 0 and self.cached_steps >= self.max_cached:
            return False
        if self.max_cont >= 0 and self.cont >= self.max_cont:
            return False
        if self.scm and self.scm in SCM_POLICIES:
            pat = SCM_POLICIES[self.scm]
            if pat[self.step % len(pat)] == 1:
                return False
        return True

    def on_stack(self, stack: BlockStack) -> tuple:
        self._switch_branch(stack.branch)
        L, states = stack.num_blocks, stack.states
        Fn, Bn = min(self.Fn, L), min(self.Bn, max(0, L - self.Fn))
        first_in = states[0].clone()
        states = stack.run(states, 0, Fn)
        fn_res = states[0] - first_in
        use_cache = False
        if self.prev_fn_res is not None and self.mid_res is not None and self._may_cache() \
                and self.prev_fn_res.shape == fn_res.shape:
            if self.state is None:
                self.state = fused.RelL1State(fn_res.device, None, self.thresh)
            self.state.reset()
            fused.rel_l1_update(fn_res.contiguous(), self.prev_fn_res, self.state)
            use_cache = bool(self.state.state[2].item() > 0.5)
        if use_cache:
            if self.use_taylor and self.seers and self.seers[0].derivs:
                states = tuple(s.add_(seer.predict(self.step)) for s, seer in zip(states, self.seers))
            else:
                states = tuple(s.add_(r) for s, r in zip(states, self.mid_res))
            self.cached_steps += 1
            self.cont += 1
            self.stats["skipped_steps"] += 1
            self.stats["skipped_blocks"] += L - Fn - Bn
            self.stats["computed_blocks"] += Fn + Bn
        else:
            before = tuple(s.clone() for s in states)
            states = stack.run(states, Fn, L - Bn)
            self.mid_res = tuple(o - b for o, b in zip(states, before))
            self.prev_fn_res = fn_res.contiguous()
            if self.use_taylor:
                if len(self.seers) != len(states):
                    self.seers = [TaylorSeer(self.order) for _ in states]
                for seer, r in zip(self.seers, self.mid_res):
                    seer.update(r, self.step)
            self.cont = 0
            self.stats["computed_blocks"] += L
        if Bn:
            states = stack.run(states, L - Bn, L)
        self.step += 1
        self.stats["steps"] += 1
        return states

    def _hook(self, model, run_blocks, img, txt, mods, cos, sin, kv_lens, ws, temb):
        """Qwen-Image entry: blocks run in place on the two streams."""
        def run(states, a, b):
            if b > a:
                run_blocks(img, txt, mods, cos, sin, kv_lens, ws, a, b)
            return (img, txt)
        return self.on_stack(BlockStack(model.cfg.num_layers, (img, txt), None, run))
