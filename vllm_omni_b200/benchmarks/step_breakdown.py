"""Where one denoising step of the flagship DiT spends its device time, by native entry point.

    python -m vllm_omni_b200.benchmarks.step_breakdown --layers 60 --steps 2

    python -m torch.distributed.run --nproc-per-node P --master-addr 127.0.0.1 --master-port 29555 \
        -m vllm_omni_b200.benchmarks.step_breakdown --layers 8 --batch 1        (fused Ulysses over P GPUs)

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
    import os
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    cfg = QwenImageTransformerConfig(num_layers=a.layers)
    torch.manual_seed(0)
    model = QwenImageTransformer2DModel(cfg, dtype=torch.bfloat16, device=dev)
    if world > 1:
        # sequence parallel over all ranks: every rank keeps S/P image rows and L/P text rows
        from vllm_omni_b200.parallel import parallel_state as ps
        from vllm_omni_b200.parallel.ulysses import UlyssesJointAttention
        ps.init_distributed_environment(world_size=world, rank=rank, local_rank=local_rank, backend="nccl")
        ps.initialize_model_parallel(sequence_parallel_size=world, ulysses_degree=world, backend="nccl")
        model.sp = UlyssesJointAttention(ps.get_sp_group().ulysses, cfg.num_attention_heads, cfg.attention_head_dim,
                                         mode=os.environ.get("OMNI_SP_MODE"))
    S = (a.height // 16) * (a.width // 16)
    g = torch.Generator(device="cpu").manual_seed(0)
    x = torch.randn(a.batch, S, cfg.in_channels, generator=g).to(dev, torch.bfloat16)
    e = torch.randn(a.batch, a.text_len, cfg.joint_attention_dim, generator=g).to(dev, torch.bfloat16)
    t = torch.full((a.batch,), 0.5, device=dev)
    if world > 1:
        x = x[:, rank * (S // world):(rank + 1) * (S // world)].contiguous()
        Lr = a.text_len // world
        e = e[:, rank * Lr:(rank + 1) * Lr].contiguous()
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
        raw = [(n, e0.elapsed_time(e1) * 1e3) for n, e0, e1 in (nv._timing or [])]
        gaps = [(raw_prev[2].elapsed_time(cur[1]) * 1e3) for raw_prev, cur in zip(nv._timing or [], (nv._timing or [])[1:])]
        summ = nv.kernel_timing_summary()
        nv.enable_kernel_timing(False)
    tot = sum(d["total_ms"] for d in summ.values())
    rows = {k: {"launches": d["launches"] // a.steps, "ms_per_step": round(d["total_ms"] / a.steps, 3),
                "share": round(d["total_ms"] / tot, 4), "mean_us": round(d["mean_us"], 1)}
            for k, d in sorted(summ.items(), key=lambda kv: -kv[1]["total_ms"])}
    # launch sequence of one block in the middle of the last step: entry point, device us, idle us before it
    att = [i for i, (n, _) in enumerate(raw) if n.startswith("omni_attn_fwd")]
    seq = []
    if len(att) >= 3:
        mid = len(att) // 2
        for i in range(att[mid - 1] + 1, att[mid] + 1):
            seq.append([raw[i][0], round(raw[i][1], 1), round(gaps[i - 1], 1) if i >= 1 else 0.0])
    if world > 1:
        torch.distributed.barrier()
    if rank != 0:
        return
    print(json.dumps({"world": world, "layers": a.layers, "batch": a.batch, "seq": S + a.text_len, "wall_ms_per_step": round(wall * 1e3, 2),
                      "kernel_ms_per_step": round(tot / a.steps, 2), "by_entry_point": rows,
                      "one_block_sequence": seq}))


if __name__ == "__main__":
    main()
