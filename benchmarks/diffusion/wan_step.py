"""One denoiser forward of the Wan 2.2 14B geometry (40 layers, 40 heads x 128, FFN 13824) on ONE GPU at
the published video shape: 81 frames of 720 x 1280 = a 21 x 90 x 160 latent = 75,600 tokens after the
(1, 2, 2) patching.  Random weights, synthetic latents and text states; CUDA events around each forward,
median over the timed ones.  A full video is 2 (guidance branches) x steps of these.

    python benchmarks/diffusion/wan_step.py                       # the full shape, 1 warm-up + 2 timed
    python benchmarks/diffusion/wan_step.py --frames 17 --height 480 --width 832 --layers 8
    python benchmarks/diffusion/wan_step.py --device cpu --tiny   # plumbing check without a GPU"""
import argparse
import json
import os
import statistics
import sys
import time

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from vllm_omni_b200.diffusion.models.wan.transformer import WanTransformer3DModel, WanTransformerConfig


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--frames", type=int, default=81)
    ap.add_argument("--height", type=int, default=720)
    ap.add_argument("--width", type=int, default=1280)
    ap.add_argument("--text-len", type=int, default=512)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--iters", type=int, default=2)
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--tiny", action="store_true")
    a = ap.parse_args(argv)
    cfg = WanTransformerConfig()
    if a.tiny:
        cfg = WanTransformerConfig(num_attention_heads=2, attention_head_dim=24, text_dim=32, ffn_dim=64, num_layers=1)
        a.frames, a.height, a.width, a.text_len = 5, 32, 32, 8
    if a.layers:
        cfg.num_layers = a.layers
    dev = torch.device(a.device)
    dt = torch.bfloat16 if dev.type == "cuda" else torch.float32
    torch.manual_seed(0)
    model = WanTransformer3DModel(cfg, dt, dev)
    T, H, W = (a.frames - 1) // 4 + 1, a.height // 8, a.width // 8
    pt, ph, pw = cfg.patch_size
    tokens = (T // pt) * (H // ph) * (W // pw)
    lat = torch.randn(1, cfg.in_channels, T, H, W, device=dev, dtype=dt)
    txt = torch.randn(1, a.text_len, cfg.text_dim, device=dev, dtype=dt)
    ts = torch.full((1,), 500.0, device=dev)
    times = []
    with torch.no_grad():
        for i in range(a.warmup + a.iters):
            if dev.type == "cuda":
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                e0.record()
                out = model(lat, ts, txt)
                e1.record()
                torch.cuda.synchronize()
                ms = e0.elapsed_time(e1)
            else:
                t0 = time.perf_counter()
                out = model(lat, ts, txt)
                ms = (time.perf_counter() - t0) * 1e3
            if i >= a.warmup:
                times.append(ms)
    D, L, F = cfg.inner_dim, cfg.num_layers, cfg.ffn_dim
    # per layer: self-attention 4 S^2 D, q/k/v/o 8 S D^2, cross-attention q/o 4 S D^2 + 4 S Lt D, FFN 4 S D F
    flops = L * (4 * tokens * tokens * D + 12 * tokens * D * D + 4 * tokens * a.text_len * D + 4 * tokens * D * F)
    ms = statistics.median(times)
    print(json.dumps({"case": "wan_forward", "tokens": tokens, "layers": L, "ms": round(ms, 2), "all_ms": [round(t, 2) for t in times],
                      "tflops": round(flops / ms / 1e9, 1), "finite": bool(torch.isfinite(out.float()).all()),
                      "mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1) if dev.type == "cuda" else None}))


if __name__ == "__main__":
    main()
