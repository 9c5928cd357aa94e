"""Reference arm of the headline benchmark: the UNMODIFIED reference files installed under
``baseline/_ref`` drive the same metric (Qwen-Image-style 60x3072 MMDiT, 1024x1024, 50 steps,
true CFG 4.0, bf16, random-init weights, synthetic inputs).

What runs, all of it the reference's own code:
  * ``vllm_omni/diffusion/models/qwen_image/qwen_image_transformer.py`` (the DiT, vLLM parallel
    linears + RMSNorm, its attention layer with the SDPA backend the reference selects on cc 10.0),
  * ``vllm_omni/diffusion/distributed/parallel_state.py`` (world / SP / CFG groups over NCCL),
  * ``vllm_omni/diffusion/hooks/sequence_parallel.py`` (the ``_sp_plan`` split / gather hooks) and
    ``vllm_omni/diffusion/attention/parallel/ulysses.py`` (all-to-all around attention),
  * ``vllm_omni/diffusion/models/qwen_image/cfg_parallel.py`` ``QwenImageCFGParallelMixin.diffuse``
    (the denoising loop: cond + uncond forward or CFG-parallel all-gather, guidance mix with norm
    rescale, scheduler step, broadcast),
  * ``vllm_omni/diffusion/compile.py`` ``regionally_compile`` (the reference compiles the repeated
    block unless ``enforce_eager``; a compile failure falls back to eager exactly as its model
    runner does).

What does not run: the text encoder (inputs are encoder states, as the benchmark config says)
and the VAE decode, because ``diffusers`` (VAE, image processor) cannot be installed offline.
The record says so in ``reference_scope``; the VAE is about 0.2 % of this framework's own image time.

The reference package's ``__init__`` patches vLLM 0.16 internals that vLLM 0.22 no longer has
(``vllm.inputs.data``), so the top-level package and the ``qwen_image`` sub-package are entered as
bare namespace stubs (a module object with ``__path__``): their ``__init__.py`` is skipped, every
other file is imported from disk unchanged.  Third-party modules that the wheelhouse lacks
(``aenum``, and the four ``diffusers`` classes the transformer and the loop touch) are stand-ins
under ``baseline/shims``.
"""
from __future__ import annotations

import importlib
import json
import os
import sys
import time
import traceback
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.path.join(HERE, "_ref")
SHIMS = os.path.join(HERE, "shims")


def _stub_package(name: str, rel: str):
    pkg = types.ModuleType(name)
    pkg.__path__ = [os.path.join(REF_ROOT, "vllm_omni", rel) if rel else os.path.join(REF_ROOT, "vllm_omni")]
    sys.modules[name] = pkg
    return pkg


def import_reference():
    """Import the reference's DiT-path modules; returns a namespace of what the arm uses."""
    if not os.path.isdir(os.path.join(REF_ROOT, "vllm_omni")):
        raise RuntimeError("baseline/_ref/vllm_omni is missing (pip install --no-deps --target baseline/_ref not done)")
    for p in (SHIMS, REF_ROOT):
        if p not in sys.path:
            sys.path.insert(0, p)
    _stub_package("vllm_omni", "")
    importlib.import_module("vllm_omni.diffusion.models")
    q = _stub_package("vllm_omni.diffusion.models.qwen_image", os.path.join("diffusion", "models", "qwen_image"))
    sys.modules["vllm_omni.diffusion.models"].qwen_image = q
    ns = types.SimpleNamespace()
    ns.transformer = importlib.import_module("vllm_omni.diffusion.models.qwen_image.qwen_image_transformer")
    ns.cfg = importlib.import_module("vllm_omni.diffusion.models.qwen_image.cfg_parallel")
    ns.pstate = importlib.import_module("vllm_omni.diffusion.distributed.parallel_state")
    ns.data = importlib.import_module("vllm_omni.diffusion.data")
    ns.fctx = importlib.import_module("vllm_omni.diffusion.forward_context")
    ns.hooks = importlib.import_module("vllm_omni.diffusion.hooks.sequence_parallel")
    ns.sp_plan = importlib.import_module("vllm_omni.diffusion.distributed.sp_plan")
    ns.compile = importlib.import_module("vllm_omni.diffusion.compile")
    return ns


def _calculate_shift(image_seq_len, base_seq_len=256, max_seq_len=8192, base_shift=0.5, max_shift=0.9):
    m = (max_shift - base_shift) / (max_seq_len - base_seq_len)
    return image_seq_len * m + (base_shift - m * base_seq_len)


def run(args, par: dict, ClockSampler) -> dict:
    """Runs the reference loop and returns the JSON record (rank 0) or None (other ranks)."""
    import numpy as np
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29611")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("LOCAL_RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)

    ref = import_reference()
    from diffusers.schedulers.scheduling_flow_match_euler_discrete import FlowMatchEulerDiscreteScheduler
    from vllm.config import CompilationConfig, VllmConfig, set_current_vllm_config

    pc = ref.data.DiffusionParallelConfig(
        ulysses_degree=par.get("ulysses_degree", 1), ring_degree=par.get("ring_degree", 1),
        cfg_parallel_size=par.get("cfg_parallel_size", 1), tensor_parallel_size=par.get("tensor_parallel_size", 1),
        sequence_parallel_size=par.get("ulysses_degree", 1) * par.get("ring_degree", 1))
    od = ref.data.OmniDiffusionConfig(model="QwenImagePipeline-random-init", dtype=torch.bfloat16, parallel_config=pc,
                                      num_gpus=world)
    vcfg = VllmConfig(compilation_config=CompilationConfig())
    vcfg.parallel_config.tensor_parallel_size = pc.tensor_parallel_size

    # --- the reference worker's init_device(), restated call for call (diffusion_worker.py:86-126)
    with ref.fctx.set_forward_context(vllm_config=vcfg, omni_diffusion_config=od), set_current_vllm_config(vcfg):
        ref.pstate.init_distributed_environment(world_size=world, rank=rank)
        ref.pstate.initialize_model_parallel(
            data_parallel_size=1, cfg_parallel_size=pc.cfg_parallel_size,
            sequence_parallel_size=pc.sequence_parallel_size, ulysses_degree=pc.ulysses_degree,
            ring_degree=pc.ring_degree, tensor_parallel_size=pc.tensor_parallel_size, pipeline_parallel_size=1)
        try:
            from vllm.v1.worker.workspace import init_workspace_manager
            init_workspace_manager(dev)
        except Exception:  # noqa: BLE001  (not present in every vLLM)
            pass
        torch.manual_seed(0)
        with torch.device(dev):
            prev = torch.get_default_dtype()
            torch.set_default_dtype(torch.bfloat16)
            try:
                model = ref.transformer.QwenImageTransformer2DModel(od_config=od, num_layers=args.layers)
            finally:
                torch.set_default_dtype(prev)
    model = model.to(device=dev, dtype=torch.bfloat16).eval()
    g = torch.Generator(device=dev).manual_seed(7)
    with torch.no_grad():
        for p in model.parameters():           # uninitialised vLLM linears: fill with small finite values
            p.copy_(torch.randn(p.shape, generator=g, device=dev, dtype=torch.float32).mul_(0.02).to(p.dtype))

    # --- sequence-parallel hooks exactly as the reference's registry applies them (registry.py:195-248)
    if pc.sequence_parallel_size > 1:
        plan = ref.sp_plan.get_sp_plan_from_model(model)
        spc = ref.sp_plan.SequenceParallelConfig(ulysses_degree=pc.ulysses_degree, ring_degree=pc.ring_degree)
        ref.hooks.apply_sequence_parallel(model, spc, plan)

    compiled = "eager"
    if not getattr(args, "ref_eager", False):
        try:
            model = ref.compile.regionally_compile(model, dynamic=True)
            compiled = "regional torch.compile (reference default)"
        except Exception as e:  # noqa: BLE001  (the reference logs and continues in eager mode)
            compiled = f"eager (torch.compile failed: {type(e).__name__})"

    class Loop(ref.cfg.QwenImageCFGParallelMixin):
        """Carrier of the attributes ``diffuse`` reads; the loop body is the reference's."""
        interrupt = False

        def __init__(self, transformer, scheduler):
            self.transformer = transformer
            self.scheduler = scheduler
            self._current_timestep = None

    B, L, Dj = args.batch, args.text_len, 3584
    hl, wl = args.height // 16, args.width // 16
    S_img = hl * wl
    sched = FlowMatchEulerDiscreteScheduler()
    loop = Loop(model, sched)
    gh = torch.Generator().manual_seed(1234)
    pos_h = torch.randn(B, L, Dj, generator=gh).bfloat16().pin_memory()
    neg_h = torch.randn(B, L, Dj, generator=gh).bfloat16().pin_memory()
    lat_h = torch.randn(B, S_img, 64, generator=gh).bfloat16().pin_memory()
    out_h = torch.empty(B, S_img, 64, dtype=torch.bfloat16).pin_memory()
    mask = torch.ones(B, L, dtype=torch.long, device=dev)
    img_shapes = [[(1, hl, wl)]] * B
    sigmas = np.linspace(1.0, 1.0 / args.num_inference_steps, args.num_inference_steps)
    mu = _calculate_shift(S_img)

    def image(pos, neg, lat):
        sched.set_timesteps(sigmas=sigmas, device=dev, mu=mu)
        with torch.no_grad(), ref.fctx.set_forward_context(vllm_config=vcfg, omni_diffusion_config=od), \
                set_current_vllm_config(vcfg):
            return loop.diffuse(
                prompt_embeds=pos, prompt_embeds_mask=mask, negative_prompt_embeds=neg,
                negative_prompt_embeds_mask=mask, latents=lat, img_shapes=img_shapes, txt_seq_lens=[L] * B,
                negative_txt_seq_lens=[L] * B, timesteps=sched.timesteps, do_true_cfg=True, guidance=None,
                true_cfg_scale=args.cfg_scale, image_latents=None, cfg_normalize=True,
                additional_transformer_kwargs={"return_dict": False, "attention_kwargs": None})

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    pos_d, neg_d, lat_d = pos_h.to(dev), neg_h.to(dev), lat_h.to(dev)
    try:
        out = image(pos_d, neg_d, lat_d)
    except Exception as e:  # noqa: BLE001
        if not compiled.startswith("regional"):
            raise
        # A compile error surfaces at the first call.  The reference's model runner keeps eager mode
        # when compilation fails; do the same: drop the compiled wrappers and run the blocks eagerly.
        for m in model.modules():
            if getattr(m, "_compiled_call_impl", None) is not None:
                m._compiled_call_impl = None
        compiled = f"eager (regional torch.compile failed at first call: {type(e).__name__}: {str(e)[:120]})"
        out = image(pos_d, neg_d, lat_d)
    for _ in range(max(args.warmup - 1, 0)):
        out = image(pos_d, neg_d, lat_d)
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    for s, e in ev:
        s.record()
        out = image(pos_d, neg_d, lat_d)
        e.record()
    barrier()
    dev_ms = sum(s.elapsed_time(e) for s, e in ev) / args.steps
    assert torch.isfinite(out.float()).all(), "reference loop produced non-finite latents"

    # end to end: inputs from pinned host memory every step, final latents read back
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        o = image(pos_h.to(dev, non_blocking=True), neg_h.to(dev, non_blocking=True), lat_h.to(dev, non_blocking=True))
        out_h.copy_(o, non_blocking=True)
        torch.cuda.synchronize()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    clocks = sampler.stop()

    t = torch.tensor([dev_ms, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = float(t[0]), float(t[1])
    if rank != 0:
        return None
    s_img = dev_ms / 1e3 / B
    return {
        "metric": "qwen_image_1024_s_per_image", "value": round(s_img, 4), "unit": "s/img", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dev_ms, 2), "higher_is_better": False,
        "scaling": "strong", "vs_baseline": round(s_img / 20.0, 4), "dtype": "bf16",
        "data": "synthetic (N(0,1) text-encoder states and latents; random-init weights)",
        "impl": "reference",
        "reference_scope": "transformer denoising loop (reference QwenImageCFGParallelMixin.diffuse: 50 steps x "
                           "(cond+uncond), CFG mix + norm rescale, Euler step); no text encoder, no VAE decode "
                           "(diffusers is not installable offline)",
        "reference_mode": compiled,
        "same_config": {"layers": args.layers, "hidden": 3072, "heads": "24x128", "image_tokens": S_img,
                        "text_tokens": L, "num_inference_steps": args.num_inference_steps,
                        "true_cfg_scale": args.cfg_scale, "batch": B, "attention_backend": "SDPA (reference's "
                        "choice on compute capability 10.0)"},
        "config": {"model": f"Qwen-Image-style MMDiT {args.layers}x3072 (20B at 60 layers), 24 heads x 128",
                   "global_batch": B, "seq_len": S_img + L, "image": f"{args.height}x{args.width}",
                   "num_inference_steps": args.num_inference_steps, "true_cfg_scale": args.cfg_scale,
                   "parallelism": args.parallelism or "reference layout: see par",
                   "par": par, "l2": "inputs+weights (40 GB) exceed L2; no explicit flush",
                   "step_definition": "one full image: 50 denoise steps x (cond+uncond), no VAE"},
        "clocks": clocks,
        "e2e": {"value": round(e2e_ms / 1e3 / B, 4), "unit": "s/img",
                "h2d_bytes_per_step": int(pos_h.nbytes + neg_h.nbytes + lat_h.nbytes),
                "d2h_bytes_per_step": int(out_h.nbytes)},
    }


def main(args, par, ClockSampler) -> int:
    rank = int(os.environ.get("RANK", "0"))
    try:
        rec = run(args, par, ClockSampler)
    except BaseException as e:  # noqa: BLE001
        tb = traceback.format_exc().strip().splitlines()
        where = next((ln.strip() for ln in reversed(tb) if ln.strip().startswith("File ")), "")
        if rank == 0:
            print(json.dumps({"impl": "reference",
                              "unavailable": f"{type(e).__name__}: {str(e)[:300]} [{where[:200]}]".replace("\n", " ")}),
                  flush=True)
        sys.stderr.write("\n".join(tb[-30:]) + "\n")
        sys.stdout.flush()
        os._exit(0)
    if rank == 0 and rec is not None:
        print(json.dumps(rec), flush=True)
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)
