"""Every fused compute + collective kernel timed in isolation against its local twin and its roofline.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29560 \
        -m vllm_omni_b200.benchmarks.fused_paths [--reps 20] [--rows 2048]
    python -m vllm_omni_b200.benchmarks.fused_paths --single            (fp8 GEMM and the MoE chain, one GPU)

Shapes are one rank's share of the Qwen-Image-style block (hidden 3072, 24 heads x 128) at ``--rows``
image rows per rank, and of the Qwen3-Omni thinker for the tensor-parallel and MoE cases.  Every
number is device time (CUDA events on the launching stream, a group barrier before each repetition,
median over ``--reps``, max over ranks); L2 is flushed between repetitions.  The roofline of a fused
path is the slower of its FLOPs at the measured GEMM peak and its NVLink bytes at the measured peer
copy bandwidth; the fraction reported is roofline time / measured time.

Paths (rank 0 prints one JSON line):
  qkv_scatter     QKV projection whose epilogue stores head groups into the owner ranks' buffers
                  (+ arrival signal)            vs the same GEMM with a local output
  attn_scatter    attention whose epilogue stores output rows into the owner ranks' buffers
                                                vs the same attention with a local output
  tp_row_reduce   row-parallel GEMM with the reduce-scatter in its epilogue + local reduce + peer gather
                                                vs GEMM + NCCL all-reduce
  peer_kv_attn    attention reading K/V of the peer through plain TMA loads   vs local K/V
  ring_gather_attn_single / _overlap   the ring path as built (parallel/ring.py): the peers' K/V pulled once into
                  local memory, then one launch over all keys / own shard during the pull plus a continuation
                  launch                        vs one launch over all keys held locally
  cfg_exchange    guidance mix + Euler step reading the partner's prediction over NVLink  vs local
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch

PEAK_TFLOPS, NVLINK_GBS = 1683.8, 770.0       # measured on this pool: cuBLAS bf16 burst, peer copy per direction


def _time(fn, reps, group=None, flush=None):
    ts = []
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    for _ in range(reps):
        if flush is not None:
            flush.zero_()
        if group is not None:
            group.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3)      # microseconds
    t = torch.tensor([statistics.median(ts)], device="cuda", dtype=torch.float64)
    if group is not None and group.world_size > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX, group=group.device_group)
    return float(t)


def _entry(us, flops=0.0, link_bytes=0.0, local_us=None):
    roof_us = max(flops / (PEAK_TFLOPS * 1e12), link_bytes / (NVLINK_GBS * 1e9)) * 1e6
    d = {"us": round(us, 1), "roofline_us": round(roof_us, 1), "fraction_of_roofline": round(roof_us / us, 3) if us else None,
         "tflops": round(flops / us / 1e6, 1) if flops else None, "link_GBs": round(link_bytes / us / 1e3, 1) if link_bytes else None}
    if local_us is not None:
        d["local_twin_us"] = round(local_us, 1)
    return d


def multi(a):
    from vllm_omni_b200.diffusion.layers.linear import FusedLinear
    from vllm_omni_b200.ops import attention as A
    from vllm_omni_b200.ops import fused, gemm
    from vllm_omni_b200.parallel import parallel_state as ps
    from vllm_omni_b200.parallel.peer_memory import PeerArena, SignalChannel, tensor_from_ptr
    from vllm_omni_b200.parallel.tensor_parallel import RowParallelReduce
    world, rank, lr = int(os.environ["WORLD_SIZE"]), int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    ps.init_distributed_environment(world_size=world, rank=rank, local_rank=lr, backend="nccl")
    ps.initialize_model_parallel(sequence_parallel_size=world, ulysses_degree=world, backend="nccl")
    grp = ps.get_sp_group().ulysses
    P, bf = world, torch.bfloat16
    D, H, Dh = 3072, 24, 128
    M = a.rows
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    torch.manual_seed(rank)
    out = {}

    # ---- qkv_scatter
    x = torch.randn(M, D, device=dev, dtype=bf)
    w = torch.randn(3 * D, D, device=dev, dtype=bf) * 0.02
    b = torch.zeros(3 * D, device=dev, dtype=bf)
    G = (H // P) * Dh
    arena = PeerArena(grp, (P * M * 3 * G + 4 * M * D) * 2 + (1 << 20), dev)
    joint = arena.alloc((P * M, 3 * G), bf)
    ch = SignalChannel(arena)
    grp.barrier()
    sc = (P, G, joint.peer_ptrs(rank * M * 3 * G * 2), 3 * G)
    waiter = torch.zeros(8, 3 * G, device=dev, dtype=bf)
    local = torch.empty(M, 3 * D, device=dev, dtype=bf)

    def f_scatter():
        gemm.linear(x, w, b, scatter=sc, sync=ch.signal())
        # the consumer of the arrivals (a few rows are enough to run the wait and keep the counters in step)
        fused.qk_norm_rope_(waiter.view(1, 8, -1), H // P, H // P, Dh, sync=ch.wait())
    t_sc = _time(f_scatter, a.reps, grp, flush)
    t_lo = _time(lambda: gemm.linear(x, w, b, out=local), a.reps, grp, flush)
    out["qkv_scatter"] = _entry(t_sc, 2.0 * M * 3 * D * D, M * 3 * D * 2 * (P - 1) / P, t_lo)

    # ---- attn_scatter: this rank's heads over all rows, output rows to their owners
    S = P * M
    qkv = torch.randn(1, S, 3, H // P, Dh, device=dev, dtype=bf)
    o_sym = arena.alloc((1, M, H * Dh), bf)
    ch2 = SignalChannel(arena)
    grp.barrier()
    hoff = rank * G * 2
    scat = dict(n_peers=P, rows_per_rank=M, rows_per_rank2=1, split=S, o_ptrs=o_sym.peer_ptrs(hoff), o2_ptrs=o_sym.peer_ptrs(hoff),
                o_strides=(H * Dh, Dh, M * H * Dh), o2_strides=(H * Dh, Dh, M * H * Dh))
    o_loc = torch.empty(1, S, H // P, Dh, device=dev, dtype=bf)
    wout = torch.randn(64, H * Dh, device=dev, dtype=bf) * 0.02
    probe = torch.empty(M, 64, device=dev, dtype=bf)

    def f_attn_sc():
        A.attention(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], scatter=scat, sync=ch2.signal())
        gemm.linear(o_sym.local.view(M, H * Dh), wout, out=probe, sync=ch2.wait())     # consumer of the arrivals
    t_probe = _time(lambda: gemm.linear(o_sym.local.view(M, H * Dh), wout, out=probe), a.reps, grp, flush)
    t_asc = _time(f_attn_sc, a.reps, grp, flush) - t_probe
    t_alo = _time(lambda: A.attention(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], out=o_loc), a.reps, grp, flush)
    out["attn_scatter"] = _entry(t_asc, 4.0 * (H // P) * S * S * Dh, S * G * 2 * (P - 1) / P, t_alo)

    # ---- peer_kv_attn: my queries against the peer's K/V (plain TMA loads of peer memory)
    kv_sym = arena.alloc((1, M, 2, H, Dh), bf)
    kv_sym.local.normal_()
    q_loc = torch.randn(1, M, H, Dh, device=dev, dtype=bf)
    o2 = torch.empty(1, M, H, Dh, device=dev, dtype=bf)
    grp.barrier()
    peer = tensor_from_ptr(kv_sym.ptrs[(rank + 1) % P], (1, M, 2, H, Dh), bf, dev)
    t_pkv = _time(lambda: A.attention(q_loc, peer[:, :, 0], peer[:, :, 1], out=o2), a.reps, grp, flush)
    t_lkv = _time(lambda: A.attention(q_loc, kv_sym.local[:, :, 0], kv_sym.local[:, :, 1], out=o2), a.reps, grp, flush)
    out["peer_kv_attn"] = _entry(t_pkv, 4.0 * H * M * M * Dh, M * 2 * H * Dh * 2, t_lkv)

    # ---- ring_gather_attn: the sequence-parallel ring as built (parallel/ring.py): own-chunk attention while a
    # side stream pulls the peers' K/V into local memory, then the continuation launch that combines both
    from vllm_omni_b200.parallel.ring import RingJointAttention
    ring = RingJointAttention(grp, H, Dh, "peer")
    ring.setup(1, M, 0, dev, bf)
    ring.qkv_local.normal_()
    grp.barrier()
    kv_full = torch.randn(1, P * M, 2, H, Dh, device=dev, dtype=bf)
    t_full = _time(lambda: A.attention(q_loc, kv_full[:, :, 0], kv_full[:, :, 1], out=o2), a.reps, grp, flush)
    for mode in ("single", "overlap"):
        os.environ["OMNI_RING_MODE"] = mode
        ring._side = None
        t_ring = _time(lambda: ring.attend(None, None), a.reps, grp, flush)
        key = f"ring_gather_attn_{mode}"
        out[key] = _entry(t_ring, 4.0 * H * M * (P * M) * Dh, (P - 1) * M * 2 * H * Dh * 2, t_full)
        out[key]["local_twin"] = "one attention launch over all P*M keys held locally"
    os.environ.pop("OMNI_RING_MODE", None)
    ring.close()

    # ---- tp_row_reduce: MLP down-projection, K sharded over the ranks
    Kp = 4 * D // P
    lin = FusedLinear(Kp, D, bias=False, dtype=bf, device=dev)
    hcol = torch.randn(M, Kp, device=dev, dtype=bf)
    resid = torch.randn(M, D, device=dev, dtype=bf)
    red_peer, red_nccl = RowParallelReduce(grp, "peer"), RowParallelReduce(grp, "nccl")
    t_peer = _time(lambda: red_peer.linear(lin, hcol, residual=resid), a.reps, grp, flush)
    t_nccl = _time(lambda: red_nccl.linear(lin, hcol, residual=resid), a.reps, grp, flush)
    # reduce-scatter in + all-gather out: 2 (P - 1) / P of the [M, D] activation per rank and direction
    out["tp_row_reduce"] = _entry(t_peer, 2.0 * M * D * Kp, 2 * M * D * 2 * (P - 1) / P, t_nccl)
    out["tp_row_reduce"]["local_twin"] = "GEMM + NCCL all-reduce + eager residual add"

    # ---- cfg_exchange (pairs of ranks): velocity of the partner read over NVLink inside the step kernel
    if P == 2:
        from vllm_omni_b200.parallel.cfg_parallel import CFGExchange
        ex = CFGExchange(grp)
        v = torch.randn(1, 4096, 64, device=dev, dtype=bf)
        lat = torch.randn(1, 4096, 64, device=dev)
        lo = torch.empty(1, 4096, 64, device=dev, dtype=bf)
        t_ex = _time(lambda: ex.step(v, lat, 4.0, -0.02, True, lo), a.reps, grp, None)
        t_el = _time(lambda: fused.cfg_euler_step_(v, v, lat, 4.0, -0.02, True, lo), a.reps, grp, None)
        out["cfg_exchange"] = _entry(t_ex, 0.0, v.numel() * 2, t_el)
        out["cfg_exchange"]["note"] = "includes the copy into the exchange slot and the barrier kernel; latency-bound"
        ex.close()
    red_peer.close()
    arena.close()
    if rank == 0:
        print(json.dumps({"world": P, "rows_per_rank": M, "reps": a.reps, "peaks": {"bf16_tflops": PEAK_TFLOPS,
                          "nvlink_GBs_per_direction": NVLINK_GBS}, "paths": out}))


def single(a):
    """fp8 block-scaled GEMM and the MoE chain on one GPU (no collective)."""
    from vllm_omni_b200.diffusion.quantization import fp8 as Q
    from vllm_omni_b200.ops import gemm
    from vllm_omni_b200.ops.moe import MoEWorkspace, moe_forward
    dev, bf = torch.device("cuda"), torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    out = {}
    M, N, K = 8192, 9216, 3072
    x = torch.randn(M, K, device=dev, dtype=bf)
    w = torch.randn(N, K, device=dev, dtype=bf) * 0.02
    st = Q.quantize_weight_blockwise(w)
    y = torch.empty(M, N, device=dev, dtype=bf)
    t8 = _time(lambda: Q.fp8_linear(x, st, None, out=y), a.reps, None, flush)
    t16 = _time(lambda: gemm.linear(x, w, out=y), a.reps, None, flush)
    out["fp8_gemm_8192x9216x3072"] = _entry(t8, 2.0 * M * N * K, 0.0, t16)
    out["fp8_gemm_8192x9216x3072"]["note"] = "includes the row-wise activation quantisation kernel; roofline is the bf16 peak"
    # Qwen3-Omni thinker MoE layer: 128 experts, top-8, hidden 2048, FFN 768
    E, k, Dm, F = 128, 8, 2048, 768
    w13 = torch.randn(E, 2 * F, Dm, device=dev, dtype=bf) * 0.02
    w2 = torch.randn(E, Dm, F, device=dev, dtype=bf) * 0.02
    for T in (64, 4096):
        xx = torch.randn(T, Dm, device=dev, dtype=bf)
        logits = torch.randn(T, E, device=dev, dtype=bf)
        ws = MoEWorkspace()
        t = _time(lambda: moe_forward(xx, logits, w13, w2, k, True, ws=ws), a.reps, None, flush)
        d = _entry(t, 2.0 * T * k * 3 * F * Dm)
        # decode-size batches are bound by streaming the touched experts' weights
        touched = min(E, T * k)
        d["hbm_us_for_touched_weights"] = round(touched * 3 * F * Dm * 2 / 6532.2e9 * 1e6, 1)
        out[f"moe_chain_T{T}"] = d
    print(json.dumps({"world": 1, "reps": a.reps, "paths": out}))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--rows", type=int, default=2048, help="image rows of one rank")
    ap.add_argument("--single", action="store_true")
    a = ap.parse_args(argv)
    if a.single or int(os.environ.get("WORLD_SIZE", "1")) == 1:
        return single(a)
    return multi(a)


if __name__ == "__main__":
    main()
