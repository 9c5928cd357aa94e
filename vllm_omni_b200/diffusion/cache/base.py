"""Cache backend interface (vllm_omni/diffusion/cache/base.py, selector.py): a backend wraps
the transformer's block loop and may skip blocks.

Two hook points.  ``transformer.stack_hook`` is the model-agnostic one: once per denoising step the
transformer describes its block loop as a ``BlockStack`` (number of blocks, the residual-stream
tensors entering the loop, a probe tensor for the change metric, and ``run(states, a, b)`` that applies
blocks a..b-1) and takes back the states after the loop.  ``transformer.block_hook`` is the older
Qwen-Image entry with that model's in-place block runner; the backends adapt it onto the same code.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable


@dataclass
class BlockStack:
    num_blocks: int
    states: tuple                     # residual-stream tensors entering the loop (run may update them in place)
    probe: object                     # tensor whose step-to-step change drives the skip decision
    run: Callable                     # run(states, a, b) -> states after blocks a..b-1
    branch: int = 0                   # which guidance branch this call belongs to (conditional 0, unconditional 1, ...)


class CacheBackend:
    name = "none"

    def __init__(self, config):
        self.config = config
        self.enabled = False
        self.stats = {"steps": 0, "skipped_steps": 0, "computed_blocks": 0, "skipped_blocks": 0}

    def enable(self, pipeline) -> None:
        tr = getattr(pipeline, "transformer", None)
        if tr is not None and hasattr(tr, "stack_hook"):
            tr.stack_hook = self.on_stack
        elif tr is not None and hasattr(tr, "block_hook"):
            tr.block_hook = self._hook
        else:
            raise ValueError(f"{type(pipeline).__name__} has no transformer with a block hook; "
                             f"{self.name} cannot be enabled")
        self.transformer = tr
        self.enabled = True

    def disable(self, pipeline) -> None:
        tr = pipeline.transformer
        if hasattr(tr, "stack_hook"):
            tr.stack_hook = None
        if hasattr(tr, "block_hook"):
            tr.block_hook = None
        self.enabled = False

    # attributes that hold per-request decision state; kept separately for every guidance branch, so that a
    # pipeline that calls the transformer once per branch compares each branch with its own previous step
    _branch_attrs: tuple = ()

    def _switch_branch(self, branch: int) -> None:
        cur = getattr(self, "_branch", 0)
        if branch == cur:
            return
        store = self.__dict__.setdefault("_branch_store", {})
        store[cur] = {a: getattr(self, a) for a in self._branch_attrs}
        saved = store.get(branch)
        if saved is None:
            saved = store.get("fresh") or {}
        for a, v in saved.items():
            setattr(self, a, v)
        self._branch = branch

    def on_stack(self, stack: BlockStack) -> tuple:
        return stack.run(stack.states, 0, stack.num_blocks)

    def refresh(self, pipeline, num_inference_steps: int | None = None) -> None:
        """Reset the per-request state (called before every request)."""
        self.stats = {k: 0 for k in self.stats}
        self._branch = 0
        self._branch_store = {}

    def _remember_fresh_state(self) -> None:
        """Called by subclasses at the end of ``refresh``: the state a not-yet-seen branch starts from."""
        import copy
        self._branch_store = {"fresh": {a: copy.copy(getattr(self, a)) for a in self._branch_attrs}}

    def summary(self) -> dict:
        s = dict(self.stats)
        tot = s["computed_blocks"] + s["skipped_blocks"]
        s["block_skip_ratio"] = s["skipped_blocks"] / tot if tot else 0.0
        return s

    def _hook(self, model, run_blocks, img, txt, mods, cos, sin, kv_lens, ws, temb):
        return run_blocks(img, txt, mods, cos, sin, kv_lens, ws)
