"""Single-kernel workloads for profiling and roofline reports.

    python -m vllm_omni_b200.benchmarks.kernel_cases gemm|gemm_gelu|attn|attn64|attn_sdpa|norm|qkrope|decode [--iters N]

Each case runs one kernel on the Qwen-Image 1024x1024 shapes (inputs larger than L2), prints
the CUDA-event time (median, L2 flushed between iterations) and the achieved fraction of the
measured peaks in MEASURED_PEAKS.json (fallback 1590 TFLOP/s, 6650 GB/s).
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def _peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["bf16_tflops"], d["hbm_gbs"], "measured"
    return 1590.0, 6650.0, "fallback"


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--bn", type=int, default=0, help="GEMM tile override (512 = CTA-pair kernel)")
    ap.add_argument("--impl", default=None, help="decode: tc (tcgen05, default) or simt")
    a = ap.parse_args(argv)
    from vllm_omni_b200.ops import attention as A, fused, gemm, kv_cache as KC, _native as nv
    dev = torch.device("cuda")
    torch.manual_seed(0)
    bf = torch.bfloat16
    flops = bytes_ = 0.0
    if a.case in ("gemm", "gemm_gelu", "gemm_down"):
        M, N, K = (8192, 9216, 3072) if a.case == "gemm" else ((8192, 12288, 3072) if a.case == "gemm_gelu" else (8192, 3072, 12288))
        x = torch.randn(M, K, device=dev, dtype=bf)
        w = torch.randn(N, K, device=dev, dtype=bf) * 0.02
        b = torch.zeros(N, device=dev, dtype=bf)
        out = torch.empty(M, N, device=dev, dtype=bf)
        fn = lambda: gemm.linear(x, w, b, act="gelu_tanh" if a.case == "gemm_gelu" else None, out=out, force_bn=a.bn)
        flops = 2.0 * M * N * K
    elif a.case in ("attn", "attn64", "attn_sdpa"):
        # attn: the Qwen-Image joint attention; attn64: head size 64 at the same width (48 heads);
        # attn_sdpa: torch SDPA (the library path the reference takes on this GPU) on the attn shape
        B, S = 2, 4352
        H, D = (48, 64) if a.case == "attn64" else (24, 128)
        qkv = torch.randn(B, S, 3, H, D, device=dev, dtype=bf)
        out = torch.empty(B, S, H, D, device=dev, dtype=bf)
        if a.case == "attn_sdpa":
            qt, kt, vt = (qkv[:, :, i].transpose(1, 2) for i in range(3))
            fn = lambda: torch.nn.functional.scaled_dot_product_attention(qt, kt, vt)
        else:
            fn = lambda: A.attention(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], out=out)
        flops = 4.0 * B * H * S * S * D
    elif a.case == "norm":
        x = torch.randn(2, 4096, 3072, device=dev, dtype=bf)
        mod = torch.randn(2, 6 * 3072, device=dev, dtype=bf)
        y = torch.empty_like(x)
        fn = lambda: fused.norm_modulate(x, shift=mod[:, :3072], scale=mod[:, 3072:6144], out=y)
        bytes_ = 2.0 * x.numel() * 2
    elif a.case == "qkrope":
        qkv = torch.randn(2, 4352, 3 * 3072, device=dev, dtype=bf)
        ws = [torch.ones(128, device=dev, dtype=bf) for _ in range(4)]
        ang = torch.randn(4352, 64, device=dev)
        cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
        fn = lambda: fused.qk_norm_rope_(qkv, 24, 24, 128, *ws, s_alt=4096, cos=cos, sin=sin)
        bytes_ = 2.0 * qkv.numel() * 2 * 2 / 3
    elif a.case == "decode":
        n, H, Hkv, ctx, bs = 64, 32, 4, 2048, 16
        nb = n * ctx // bs
        kc = torch.randn(nb, bs, Hkv, 128, device=dev, dtype=bf)
        vc = torch.randn_like(kc)
        bt = torch.arange(nb, dtype=torch.int32, device=dev).view(n, -1)
        sl = torch.full((n,), ctx, dtype=torch.int32, device=dev)
        q = torch.randn(n, H, 128, device=dev, dtype=bf)
        fn = lambda: KC.paged_decode(q, kc, vc, bt, sl, impl=a.impl)
        bytes_ = 2.0 * kc.numel() * 2
    elif a.case in ("vae", "vae_torch"):
        # 1024 x 1024 image: latent 16 x 128 x 128 through the full decoder
        from vllm_omni_b200.diffusion.models.vae.autoencoder_kl_qwenimage import AutoencoderKLQwenImage2d
        vae = AutoencoderKLQwenImage2d().to(dev).bfloat16()
        vae.decoder_impl = "torch" if a.case == "vae_torch" else "nhwc"
        z = torch.randn(1, 16, 128, 128, device=dev)
        fn = lambda: vae.decode(z)
        bytes_ = 0.0
    elif a.case in ("kl_vae", "kl_vae_torch"):
        # 1024 x 1024 image through the FLUX-family AutoencoderKL decoder (GroupNorm ResNet blocks)
        from vllm_omni_b200.diffusion.models.vae.autoencoder_kl import AutoencoderKL
        vae = AutoencoderKL().to(dev).bfloat16()
        vae.decoder_impl = "torch" if a.case == "kl_vae_torch" else "nhwc"
        z = torch.randn(1, 16, 128, 128, device=dev)
        fn = lambda: vae.decode(z)
        bytes_ = 0.0
    elif a.case in ("wan_vae", "wan_vae_torch"):
        # 17 frames of 480 x 832: latent 16 x 5 x 60 x 104 through the causal 3-D decoder, one latent frame per chunk
        from vllm_omni_b200.diffusion.models.vae.autoencoder_kl_wan import AutoencoderKLWan
        vae = AutoencoderKLWan().to(dev).bfloat16()
        vae.decoder_impl = "torch" if a.case == "wan_vae_torch" else "nhwc"
        z = torch.randn(1, 16, 5, 60, 104, device=dev)
        fn = lambda: vae.decode(z)
        bytes_ = 0.0
    else:
        raise SystemExit(f"unknown case {a.case}")
    flush = None if a.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(a.iters):
        if flush is not None:
            flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); fn(); e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    ms = ts[len(ts) // 2]
    tf, gbs, src = _peaks()
    rec = {"case": a.case, "ms": round(ms, 4), "status": int(nv.status_word(dev).item())}
    if flops:
        rec.update(tflops=round(flops / ms / 1e9, 1), frac_of_peak=round(flops / ms / 1e9 / tf, 3), peak=f"{tf} TFLOP/s {src}")
    if bytes_:
        rec.update(gbs=round(bytes_ / ms / 1e6, 1), frac_of_peak=round(bytes_ / ms / 1e6 / gbs, 3), peak=f"{gbs} GB/s {src}")
    print(json.dumps(rec))


if __name__ == "__main__":
    main()
