"""Command line: ``vllm-omni-b200 serve MODEL [--omni] ...`` and ``vllm-omni-b200 bench ...``
(vllm_omni/entrypoints/cli/main.py, cli/serve.py: the flag set of ``OmniServeCommand``)."""
from __future__ import annotations

import argparse
import json
import sys


def make_serve_parser(sub=None) -> argparse.ArgumentParser:
    p = (sub.add_parser("serve", help="start the OpenAI-compatible server") if sub is not None
         else argparse.ArgumentParser("serve"))
    p.add_argument("model")
    p.add_argument("--omni", action="store_true", help="accepted for compatibility; every model is served as omni")
    p.add_argument("--host", default="0.0.0.0")
    p.add_argument("--port", type=int, default=8000)
    p.add_argument("--served-model-name", default=None)
    p.add_argument("--stage-configs-path", default=None)
    p.add_argument("--stage-init-timeout", type=int, default=300)
    p.add_argument("--init-timeout", type=int, default=300)
    p.add_argument("--shm-threshold-bytes", type=int, default=65536)
    p.add_argument("--log-stats", action="store_true")
    p.add_argument("--log-file", default=None)
    p.add_argument("--batch-timeout", type=int, default=10, help="diffusion batch window in ms")
    p.add_argument("--worker-backend", default="mp", choices=["mp", "ray"])
    p.add_argument("--ray-address", default=None)
    p.add_argument("--num-gpus", type=int, default=None)
    p.add_argument("--usp", "--ulysses-degree", dest="ulysses_degree", type=int, default=1)
    p.add_argument("--ring", dest="ring_degree", type=int, default=1)
    p.add_argument("--cfg-parallel-size", type=int, default=1)
    p.add_argument("--tensor-parallel-size", "-tp", type=int, default=1)
    p.add_argument("--vae-patch-parallel-size", type=int, default=1)
    p.add_argument("--cache-backend", default="none", choices=["none", "tea_cache", "cache_dit"])
    p.add_argument("--cache-config", type=json.loads, default=None, help="JSON dict")
    p.add_argument("--enable-cache-dit-summary", action="store_true")
    p.add_argument("--vae-use-slicing", action="store_true")
    p.add_argument("--vae-use-tiling", action="store_true")
    p.add_argument("--enable-cpu-offload", action="store_true")
    p.add_argument("--enable-layerwise-offload", action="store_true")
    p.add_argument("--boundary-ratio", type=float, default=None)
    p.add_argument("--flow-shift", type=float, default=None)
    p.add_argument("--default-sampling-params", type=json.loads, default=None, help="JSON dict")
    p.add_argument("--max-generated-image-size", type=int, default=None)
    p.add_argument("--quantization", default=None, choices=[None, "fp8"])
    p.add_argument("--enforce-eager", action="store_true")
    p.add_argument("--dtype", default="bfloat16")
    p.add_argument("--lora-path", default=None)
    return p


def serve_kwargs(args) -> dict:
    from ...diffusion.data import DiffusionParallelConfig
    kw = dict(stage_configs_path=args.stage_configs_path, stage_init_timeout=args.stage_init_timeout,
              init_timeout=args.init_timeout, shm_threshold_bytes=args.shm_threshold_bytes, log_stats=args.log_stats,
              log_file=args.log_file, batch_timeout=args.batch_timeout, worker_backend=args.worker_backend,
              ray_address=args.ray_address, served_model_name=args.served_model_name)
    par = dict(ulysses_degree=args.ulysses_degree, ring_degree=args.ring_degree,
               cfg_parallel_size=args.cfg_parallel_size, tensor_parallel_size=args.tensor_parallel_size,
               vae_patch_parallel_size=args.vae_patch_parallel_size)
    if any(v != 1 for v in par.values()):
        kw["parallel_config"] = DiffusionParallelConfig(**par)
    for k in ("cache_backend", "cache_config", "vae_use_slicing", "vae_use_tiling", "enable_cpu_offload",
              "enable_layerwise_offload", "boundary_ratio", "flow_shift", "quantization", "enforce_eager", "dtype",
              "lora_path", "enable_cache_dit_summary", "num_gpus"):
        v = getattr(args, k)
        if v not in (None, False, "none"):
            kw[k] = v
    return kw


def main(argv=None) -> int:
    ap = argparse.ArgumentParser("vllm-omni-b200")
    sub = ap.add_subparsers(dest="cmd", required=True)
    make_serve_parser(sub)
    b = sub.add_parser("bench", help="benchmarks")
    b.add_argument("what", choices=["serve", "image"])
    b.add_argument("rest", nargs=argparse.REMAINDER)
    args = ap.parse_args(argv)
    if args.cmd == "serve":
        from ..openai.api_server import omni_run_server
        omni_run_server(args.model, host=args.host, port=args.port, **serve_kwargs(args))
        return 0
    if args.cmd == "bench":
        from ...benchmarks.serve_bench import main as bench_main
        return bench_main([args.what] + args.rest)
    return 1


if __name__ == "__main__":
    sys.exit(main())
