"""Where one denoising step of the flagship DiT spends its device time, by native entry point.

    python -m vllm_omni_b200.benchmarks.step_breakdown --layers 60 --steps 2

Runs the Qwen-Image-style transformer eagerly (no CUDA graph) with CUDA events around every
native launch (``ops/_native.enable_kernel_timing``) and prints one JSON line: per entry point
launches, total ms and share of the summed kernel time, plus the wall-clock time of the step.
Device timers serialise nothing and add two event records per launch, so shares are faithful
while absolute step time is a little above the graph-captured path."""
from __future__ import annotations

import argparse
import json
import time

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=60)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--height", type=int, default=1024)
    ap.add_argument("--width", type=int, default=1024)
    ap.add_argument("--text-len", type=int, default=256)
    ap.add_argument("--batch", type=int, default=2, help="2 = conditional + unconditional rows of one CFG step")
    a = ap.parse_args(argv)
    from vllm_omni_b200.diffusion.models.qwen_image.transformer import (QwenImageTransformer2DModel,
                                                                        QwenImageTransformerConfig)
    from vllm_omni_b200.ops import _native as nv
    dev = torch.device("cuda")
    cfg = QwenImageTransformerConfig(num_layers=a.layers)
    model = QwenImageTransformer2DModel(cfg, dtype=torch.bfloat16, device=dev)
    S = (a.height // 16) * (a.width // 16)
    g = torch.Generator(device="cpu").manual_seed(0)
    x = torch.randn(a.batch, S, cfg.in_channels, generator=g).to(dev, torch.bfloat16)
    e = torch.randn(a.batch, a.text_len, cfg.joint_attention_dim, generator=g).to(dev, torch.bfloat16)
    t = torch.full((a.batch,), 0.5, device=dev)
    shape = (1, a.height // 16, a.width // 16)
    with torch.no_grad():
        for _ in range(2):
            model(x, e, t, shape)
        torch.cuda.synchronize()
        nv.enable_kernel_timing(True)
        t0 = time.perf_counter()
        for _ in range(a.steps):
            model(x, e, t, shape)
        torch.cuda.synchronize()
        wall = (time.perf_counter() - t0) / a.steps
        summ = nv.kernel_timing_summary()
        nv.enable_kernel_timing(False)
    tot = sum(d["total_ms"] for d in summ.values())
    rows = {k: {"launches": d["launches"] // a.steps, "ms_per_step": round(d["total_ms"] / a.steps, 3),
                "share": round(d["total_ms"] / tot, 4), "mean_us": round(d["mean_us"], 1)}
            for k, d in sorted(summ.items(), key=lambda kv: -kv[1]["total_ms"])}
    print(json.dumps({"layers": a.layers, "batch": a.batch, "seq": S + a.text_len, "wall_ms_per_step": round(wall * 1e3, 2),
                      "kernel_ms_per_step": round(tot / a.steps, 2), "by_entry_point": rows}))


if __name__ == "__main__":
    main()
