"""Headline benchmark: Qwen-Image-style 20B MMDiT, 1024x1024, 50 flow-match Euler steps,
true CFG 4.0, bf16, random-init weights, synthetic inputs — seconds per image.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torchrun)

One "step" is one full image (50 denoising steps x cond+uncond, VAE decode).  Two numbers:
  value  device-timed (CUDA events) pipeline call on device-resident inputs;
  e2e    the same image through the public ``Omni.generate`` API, inputs copied from pinned
         host memory every step and the decoded image read back to the host.
Weights (40 GB) and activations are far larger than L2, so no explicit L2 flush is needed
between timed iterations.  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

BASELINE_S_PER_IMG = 20.0   # published "Qwen-Image 1024^2, 50 steps, no cache" (hardware not stated)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="omni", choices=["omni", "reference"])
    ap.add_argument("--height", type=int, default=1024)
    ap.add_argument("--width", type=int, default=1024)
    ap.add_argument("--num-inference-steps", type=int, default=50)
    ap.add_argument("--cfg-scale", type=float, default=4.0)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--text-len", type=int, default=256)
    ap.add_argument("--layers", type=int, default=60, help="60 = the 20B config; anything else is a smoke run")
    ap.add_argument("--parallelism", default=None, help="e.g. sp8, cfg2xsp4, tp8 (default: cfg2 at N=2, cfg2 x sp(N/2) above)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--ref-eager", action="store_true", help="reference arm: skip its regional torch.compile")
    return ap.parse_args()


def reference_arm(args):
    """Runs the unmodified reference (installed under ``baseline/_ref``) on the same metric and
    config; ``baseline/reference_arm.py`` says which of its files run.  The reference's layouts:
    N=1 single, N=2 CFG-parallel, N>=4 CFG-parallel x Ulysses N/2 (its `cfg_parallel_size` and
    `ulysses_degree` options) unless ``--parallelism`` names another."""
    from baseline import reference_arm as ra
    par = parse_parallelism(args.parallelism, args.gpus)
    return ra.main(args, par, ClockSampler)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); pw.append(float(f[3]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm), "reasons": sorted(reasons)}


def default_parallelism(n: int) -> str:
    """The two CFG branches go to two halves of the GPUs (no per-layer traffic between them);
    each half splits the sequence (fused Ulysses) when it has more than one GPU."""
    if n == 1:
        return "single"
    if n == 2:
        return "cfg2"
    return f"cfg2xsp{n // 2}" if n % 2 == 0 else f"sp{n}"


def parse_parallelism(spec: str | None, n: int) -> dict:
    if n == 1:
        return {}
    spec = (spec or default_parallelism(n)).lower()
    out = {"ulysses_degree": 1, "ring_degree": 1, "cfg_parallel_size": 1, "tensor_parallel_size": 1}
    for part in spec.split("x"):
        if part.startswith("cfg"):
            out["cfg_parallel_size"] = int(part[3:])
        elif part.startswith("sp") or part.startswith("ulysses"):
            out["ulysses_degree"] = int(part.lstrip("spulyse"))
        elif part.startswith("ring"):
            out["ring_degree"] = int(part[4:])
        elif part.startswith("tp"):
            out["tensor_parallel_size"] = int(part[2:])
    world = out["ulysses_degree"] * out["ring_degree"] * out["cfg_parallel_size"] * out["tensor_parallel_size"]
    if world != n:
        raise SystemExit(f"parallelism {spec} needs {world} GPUs, got --gpus {n}")
    return out


def main():
    args = parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    import torch
    import torch.distributed as dist
    from vllm_omni_b200.diffusion.data import DiffusionParallelConfig
    from vllm_omni_b200.entrypoints.omni import Omni
    from vllm_omni_b200.inputs import OmniDiffusionSamplingParams
    from vllm_omni_b200.ops import _native as nv

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    par = parse_parallelism(args.parallelism, args.gpus)
    tcfg = dict(num_layers=args.layers)
    omni = Omni("QwenImagePipeline", dtype="bfloat16", tf_model_config=tcfg, diffusion_load_format="dummy",
                parallel_config=DiffusionParallelConfig(**par), max_batch_size=args.batch, output_type="pil")
    stage = omni.stage_list[0]
    B, L, Dj = args.batch, args.text_len, 3584

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- synthetic inputs: text-encoder states N(0,1) in pinned host memory
    g = torch.Generator().manual_seed(1234)
    pos_h = [torch.randn(L, Dj, generator=g).bfloat16().pin_memory() for _ in range(B)]
    neg_h = [torch.randn(L, Dj, generator=g).bfloat16().pin_memory() for _ in range(B)]

    def make_sp(out_type):
        return OmniDiffusionSamplingParams(height=args.height, width=args.width,
                                           num_inference_steps=args.num_inference_steps,
                                           true_cfg_scale=args.cfg_scale, output_type=out_type)

    def e2e_image(seed):
        """Public API call: host inputs -> H2D -> 50 steps -> VAE -> D2H -> PIL."""
        prompts = [{"prompt": "", "negative_prompt": " ",
                    "prompt_embeds": pos_h[i].to(dev, non_blocking=True),
                    "negative_prompt_embeds": neg_h[i].to(dev, non_blocking=True)} for i in range(B)]
        sp = make_sp("pil")
        sp.seed = None
        outs = omni.generate(prompts, sp)
        return outs

    # ---- device-timed arm uses the engine's pipeline object directly on device-resident inputs
    from vllm_omni_b200.diffusion.request import OmniDiffusionRequest
    pipe = _find_pipeline(omni)
    pos_d = [t.to(dev) for t in pos_h]
    neg_d = [t.to(dev) for t in neg_h]

    def device_image():
        prompts = [{"prompt": "", "negative_prompt": " ", "prompt_embeds": pos_d[i],
                    "negative_prompt_embeds": neg_d[i]} for i in range(B)]
        sp = make_sp("pt")
        sp.generator = torch.Generator(device=dev).manual_seed(0)
        return pipe.forward(OmniDiffusionRequest(prompts, sp, ["bench"] * B))

    # ---- N > 1: the parallel layout against the same image computed by rank 0 alone (same weights,
    #      same seed, the full-depth model, 4 denoising steps).  The GPU test box of a driver may
    #      have one GPU only, so this is where the fused exchange kernels are checked at scale.
    check = None
    if world > 1 and not par.get("tensor_parallel_size", 1) > 1:
        def short_image():
            prompts = [{"prompt": "", "negative_prompt": " ", "prompt_embeds": pos_d[i],
                        "negative_prompt_embeds": neg_d[i]} for i in range(B)]
            sp = make_sp("pt")
            sp.num_inference_steps = 4
            sp.generator = torch.Generator(device=dev).manual_seed(0)
            return pipe.forward(OmniDiffusionRequest(prompts, sp, ["check"] * B))
        par_img = short_image().output.float()
        barrier()
        if rank == 0:
            tr = pipe.transformer
            saved = (tr.sp, pipe.cfg_exchange)
            tr.sp, pipe.cfg_exchange = None, None
            try:
                one_img = short_image().output.float()
            finally:
                tr.sp, pipe.cfg_exchange = saved
            diff = float((par_img - one_img).abs().max())
            span = float(one_img.max() - one_img.min())
            check = {"max_abs_diff_vs_single": round(diff, 5), "tolerance": 0.03, "image_value_span": round(span, 4),
                     "what": "decoded image, 4 steps, full-depth model, N-GPU layout vs rank 0 alone"}
        barrier()
        flag = torch.tensor([0 if check is None or check["max_abs_diff_vs_single"] <= check["tolerance"] else 1],
                            device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        if int(flag):
            raise SystemExit(f"parallel image differs from the single-GPU image: {check}")

    for _ in range(args.warmup):
        out = device_image()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    n0 = nv.launch_count
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    for s, e in ev:
        s.record()
        out = device_image()
        e.record()
    barrier()
    launches = nv.launch_count - n0
    dev_ms = sum(s.elapsed_time(e) for s, e in ev) / args.steps
    assert out.error is None and out.output is not None and torch.isfinite(out.output.float()).all()

    e2e_ms = None
    h2d = d2h = 0
    if not args.no_e2e:
        e2e_image(0)   # one untimed call: thread hand-off and PIL conversion warm
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            outs = e2e_image(i)
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
        h2d = B * 2 * L * Dj * 2
        d2h = B * 3 * args.height * args.width
        if rank == 0:
            assert len(outs) == B and outs[0].images[0].size == (args.width, args.height)
    clocks = sampler.stop()

    t = torch.tensor([dev_ms, e2e_ms or 0.0], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_max = float(t[0]), float(t[1])
    if rank == 0:
        s_img = dev_ms / 1e3 / B
        rec = {
            "metric": "qwen_image_1024_s_per_image", "value": round(s_img, 4), "unit": "s/img", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dev_ms, 2), "higher_is_better": False,
            "scaling": "strong", "vs_baseline": round(s_img / BASELINE_S_PER_IMG, 4), "dtype": "bf16",
            "data": "synthetic (N(0,1) text-encoder states and latents; random-init weights)",
            "impl": "omni",
            "config": {"model": f"Qwen-Image-style MMDiT {args.layers}x3072 (20B at 60 layers), 24 heads x 128",
                       "global_batch": B, "seq_len": (args.height // 16) * (args.width // 16) + L,
                       "image": f"{args.height}x{args.width}", "num_inference_steps": args.num_inference_steps,
                       "true_cfg_scale": args.cfg_scale,
                       "parallelism": args.parallelism or default_parallelism(args.gpus),
                       "l2": "inputs+weights (40 GB) exceed L2; no explicit flush",
                       "step_definition": "one full image: 50 denoise steps x (cond+uncond) + VAE decode"},
            "clocks": clocks, "gpu_launches": int(launches),
        }
        if check is not None:
            rec["correctness"] = check
        if e2e_ms is not None:
            rec["e2e"] = {"value": round(e2e_max / 1e3 / B, 4), "unit": "s/img", "h2d_bytes_per_step": h2d,
                          "d2h_bytes_per_step": d2h}
        print(json.dumps(rec), flush=True)
    omni.close()
    if world > 1 and dist.is_initialized():
        # Sub-groups whose NCCL communicator was never used (the peer-memory paths exchange their
        # handles over Gloo) can fail to shut down cleanly; the measurement is already printed, so
        # leave together and skip the interpreter's teardown of the process groups.
        torch.cuda.synchronize()
        try:
            dist.barrier()
        except Exception:   # noqa: BLE001
            pass
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    return 0


def _find_pipeline(omni):
    """The in-process stage's pipeline object (device-timed arm only)."""
    from vllm_omni_b200.entrypoints.stage_runtime import inproc_adapter
    return inproc_adapter(0).engine.engine.executor.worker.model_runner.pipeline


if __name__ == "__main__":
    sys.exit(main())
