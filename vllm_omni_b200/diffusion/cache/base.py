"""Cache backend interface (vllm_omni/diffusion/cache/base.py, selector.py): a backend wraps
the transformer's block loop through ``transformer.block_hook`` and may skip blocks."""
from __future__ import annotations


class CacheBackend:
    name = "none"

    def __init__(self, config):
        self.config = config
        self.enabled = False
        self.stats = {"steps": 0, "skipped_steps": 0, "computed_blocks": 0, "skipped_blocks": 0}

    def enable(self, pipeline) -> None:
        tr = getattr(pipeline, "transformer", None)
        if tr is None or not hasattr(tr, "block_hook"):
            raise ValueError(f"{type(pipeline).__name__} has no transformer with a block hook; "
                             f"{self.name} cannot be enabled")
        tr.block_hook = self._hook
        self.transformer = tr
        self.enabled = True

    def disable(self, pipeline) -> None:
        pipeline.transformer.block_hook = None
        self.enabled = False

    def refresh(self, pipeline, num_inference_steps: int | None = None) -> None:
        """Reset the per-request state (called before every request)."""
        self.stats = {k: 0 for k in self.stats}

    def summary(self) -> dict:
        s = dict(self.stats)
        tot = s["computed_blocks"] + s["skipped_blocks"]
        s["block_skip_ratio"] = s["skipped_blocks"] / tot if tot else 0.0
        return s

    def _hook(self, model, run_blocks, img, txt, mods, cos, sin, kv_lens, ws, temb):
        return run_blocks(img, txt, mods, cos, sin, kv_lens, ws)
