"""Qwen3-Omni three-stage pipeline under load, in process (no HTTP): Poisson arrivals under a
concurrency cap through ``AsyncOmni``; reports end-to-end text tokens/s, p50/p90/p99 time to first
token, time to first audio packet and the audio real-time factor — the second headline metric
(e2e tok/s + p50 TTFT at 64 concurrent requests).

    # full-size architecture with random weights, all three stages on GPU 0
    python benchmarks/qwen3_omni/serving_latency.py --device cuda --num-prompts 128 --max-concurrency 64 \
        --request-rate 8 --input-len 256 --max-tokens 128
    # the published configuration: 1024 text tokens + 30 s of audio features per request, 512 output tokens,
    # 64 concurrent requests with Poisson arrivals; thinker on 4 GPUs (tensor / expert parallel)
    python benchmarks/qwen3_omni/serving_latency.py --device cuda --num-prompts 128 --max-concurrency 64 \
        --request-rate 8 --input-len 1024 --audio-seconds 30 --max-tokens 512 --codec-frames 512 \
        --thinker-tp 4 --thinker-ep
    # CPU smoke run with the tiny geometry
    python benchmarks/qwen3_omni/serving_latency.py --tiny --num-prompts 6 --max-concurrency 3

Inputs are synthetic token ids; weights are random-init, so every request runs to ``max_tokens``
(``ignore_eos``), which fixes the work per request."""
import argparse
import asyncio
import json
import os
import random
import sys
import tempfile
import time

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

YAML = """
async_chunk: ASYNC_CHUNK
stage_args:
  - stage_id: 0
    stage_type: llm
    runtime: {devices: "THINKER_DEVS", max_batch_size: MAXB, process: THINKER_PROC}
    engine_args: {model_stage: thinker, model_arch: Qwen3OmniMoeForConditionalGeneration, worker_type: ar,
                  engine_output_type: latent, device: DEVICE, max_num_batched_tokens: 8192, gpu_memory_utilization: 0.55,
                  load_format: dummy, model_overrides: OVERRIDES, tensor_parallel_size: THINKER_TP,
                  enable_expert_parallel: THINKER_EP}
    final_output: true
    final_output_type: text
    default_sampling_params: {temperature: 0.0, max_tokens: MAXTOK, ignore_eos: true, detokenize: false}
  - stage_id: 1
    stage_type: llm
    runtime: {devices: "TAIL_DEV", max_batch_size: MAXB, process: STAGE_PROC}
    engine_args: {model_stage: talker, model_arch: Qwen3OmniMoeForConditionalGeneration, worker_type: ar,
                  engine_output_type: latent, device: DEVICE, gpu_memory_utilization: 0.3, load_format: dummy,
                  model_overrides: OVERRIDES}
    engine_input_source: [0]
    custom_process_input_func: vllm_omni_b200.models.stage_input_processors.qwen3_omni.thinker2talker
    default_sampling_params: {temperature: 0.9, top_k: 50, max_tokens: CODEC, seed: 1, ignore_eos: true,
                              stop_token_ids: [], detokenize: false}
  - stage_id: 2
    stage_type: llm
    runtime: {devices: "TAIL_DEV", max_batch_size: MAXB, process: STAGE_PROC}
    engine_args: {model_stage: code2wav, model_arch: Qwen3OmniMoeForConditionalGeneration, worker_type: generation,
                  engine_output_type: audio, device: DEVICE, load_format: dummy, model_overrides: OVERRIDES}
    engine_input_source: [1]
    custom_process_input_func: vllm_omni_b200.models.stage_input_processors.qwen3_omni.talker2code2wav
    final_output: true
    final_output_type: audio
"""


def _pct(xs, q):
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(round(q / 100 * (len(xs) - 1))))] if xs else None


def _stage_split(summary: dict) -> dict:
    """Per-stage totals from the orchestrator's aggregator: generation time, tokens in / out, and the
    bytes and time of the hand-offs into the stage."""
    out: dict = {}
    if not isinstance(summary, dict):
        return out
    for ev in summary.get("stages", []):
        d = out.setdefault(str(ev.get("stage_id")), {"gen_time_ms": 0.0, "tokens_in": 0, "tokens_out": 0, "requests": 0})
        d["gen_time_ms"] += float(ev.get("stage_gen_time_ms") or 0.0)
        d["tokens_in"] += int(ev.get("num_tokens_in") or 0)
        d["tokens_out"] += int(ev.get("num_tokens_out") or 0)
        d["requests"] += 1
    for tr in summary.get("transfers", []):
        to = str(tr.get("edge", "->").split("->")[-1])
        d = out.setdefault(to, {})
        d["rx_kbytes"] = d.get("rx_kbytes", 0.0) + float(tr.get("size_kbytes") or 0.0)
        d["rx_time_ms"] = d.get("rx_time_ms", 0.0) + float(tr.get("tx_time_ms") or 0.0) + float(tr.get("rx_decode_time_ms") or 0.0)
        d["device_direct"] = bool(tr.get("device_direct"))
    for d in out.values():
        for k in ("gen_time_ms", "rx_kbytes", "rx_time_ms"):
            if k in d:
                d[k] = round(d[k], 2)
    return out


async def _run(a, path):
    from vllm_omni_b200.entrypoints.async_omni import AsyncOmni
    eng = AsyncOmni("qwen3-omni-bench", stage_configs_path=path)
    rng = random.Random(a.seed)
    vocab = 400 if a.tiny else 150000
    prompts = [{"prompt_token_ids": [rng.randrange(10, vocab) for _ in range(a.input_len)]} for _ in range(a.num_prompts)]
    if a.audio_seconds > 0:
        # 100 mel frames per second of audio, N(0,1) features; one placeholder token marks where they go
        import torch
        from vllm_omni_b200.models.qwen3_omni.config import Qwen3OmniConfig
        cfg = Qwen3OmniConfig.tiny() if a.tiny else Qwen3OmniConfig()
        n_mels = cfg.audio.num_mel_bins
        g = torch.Generator().manual_seed(a.seed)
        for p in prompts:
            p["prompt_token_ids"].insert(1, cfg.audio_token_id)
            p["multi_modal_data"] = {"audio": torch.randn(n_mels, int(a.audio_seconds * 100), generator=g)}
    sem = asyncio.Semaphore(a.max_concurrency)
    recs = []

    async def one(i, p):
        async with sem:
            t0 = time.perf_counter()
            r = {"ttft": None, "ttfp": None, "tokens": 0, "audio_s": 0.0}
            async for o in eng.generate(p, request_id=f"bench-{i}"):
                now = time.perf_counter()
                if o.final_output_type == "text" and o.outputs:
                    n = len(o.outputs[0].token_ids)
                    if n and r["ttft"] is None:
                        r["ttft"] = now - t0
                    r["tokens"] = max(r["tokens"], n)
                elif o.final_output_type == "audio":
                    mm = o.multimodal_output or {}
                    if "audio" in mm:
                        if r["ttfp"] is None:
                            r["ttfp"] = now - t0
                        r["audio_s"] += mm["audio"].numel() / float(mm.get("sample_rate", 24000))
            r["latency"] = time.perf_counter() - t0
            recs.append(r)

    t0 = time.perf_counter()
    tasks = []
    live: dict = {}

    async def progress():
        while True:
            await asyncio.sleep(a.progress)
            done = len(recs)
            print(f"[{time.perf_counter() - t0:7.1f}s] finished {done}/{len(prompts)} requests, "
                  f"{sum(r['tokens'] for r in recs)} text tokens of finished requests", file=sys.stderr, flush=True)
    mon = asyncio.create_task(progress()) if a.progress > 0 else None
    for i, p in enumerate(prompts):
        tasks.append(asyncio.create_task(one(i, p)))
        if a.request_rate > 0:
            await asyncio.sleep(rng.expovariate(a.request_rate))
    timed_out = False
    if a.time_limit > 0:
        done_set, pending = await asyncio.wait(tasks, timeout=max(1.0, a.time_limit - (time.perf_counter() - t0)))
        timed_out = bool(pending)
        for t in pending:
            t.cancel()
    else:
        await asyncio.gather(*tasks)
    if mon is not None:
        mon.cancel()
    wall = time.perf_counter() - t0
    try:
        eng_stats = eng.metrics.build_summary(wall)
    except Exception:   # noqa: BLE001
        eng_stats = {}
    eng.close()
    toks = sum(r["tokens"] for r in recs)
    out = {"metric": "qwen3_omni_e2e_tok_s", "requests": len(recs), "wall_s": round(wall, 3),
           "e2e_text_tokens_per_s": round(toks / wall, 2), "requests_per_s": round(len(recs) / wall, 3),
           "audio_seconds_per_s": round(sum(r["audio_s"] for r in recs) / wall, 3),
           "ttft_s": {f"p{q}": _pct([r["ttft"] for r in recs if r["ttft"] is not None], q) for q in (50, 90, 99)},
           "audio_ttfp_s": {f"p{q}": _pct([r["ttfp"] for r in recs if r["ttfp"] is not None], q) for q in (50, 90, 99)},
           "e2el_s": {f"p{q}": _pct([r["latency"] for r in recs], q) for q in (50, 90, 99)},
           "stages": _stage_split(eng_stats), "timed_out": timed_out,
           "talkers_started_from_running_thinker": int(getattr(eng, "stream_starts", 0)),
           "config": {"tiny": a.tiny, "input_len": a.input_len, "audio_seconds": a.audio_seconds,
                      "thinker_tp": a.thinker_tp, "thinker_ep": a.thinker_ep, "tail_device": a.tail_device,
                      "stage_processes": a.stage_processes, "max_tokens": a.max_tokens, "codec_frames": a.codec_frames,
                      "max_concurrency": a.max_concurrency, "request_rate": a.request_rate, "async_chunk": a.async_chunk,
                      "data": "synthetic token ids; random-init weights"}}
    print(json.dumps(out))
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--num-prompts", type=int, default=64)
    ap.add_argument("--max-concurrency", type=int, default=64)
    ap.add_argument("--request-rate", type=float, default=0.0, help="Poisson arrivals per second (0 = all at once)")
    ap.add_argument("--input-len", type=int, default=128)
    ap.add_argument("--max-tokens", type=int, default=64)
    ap.add_argument("--codec-frames", type=int, default=64)
    ap.add_argument("--async-chunk", action="store_true")
    ap.add_argument("--thinker-layers", type=int, default=None)
    ap.add_argument("--audio-seconds", type=float, default=0.0, help="seconds of audio features (100 mel frames / s) per request")
    ap.add_argument("--thinker-tp", type=int, default=1, help="GPUs of the thinker stage (tensor parallel)")
    ap.add_argument("--thinker-ep", action="store_true", help="whole experts per rank instead of sliced FFNs")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--stage-processes", action="store_true", help="every stage in a process of its own (own interpreter lock); "
                    "the default on a GPU")
    ap.add_argument("--tail-device", type=int, default=0, help="GPU of the talker and code2wav stages (the thinker uses GPUs 0..tp-1)")
    ap.add_argument("--stage-threads", action="store_true", help="keep the stages on threads of this process on a GPU too")
    ap.add_argument("--progress", type=float, default=0.0, help="seconds between progress lines on stderr (0 = none)")
    ap.add_argument("--time-limit", type=float, default=0.0, help="stop waiting after this many seconds and report what finished")
    a = ap.parse_args(argv)
    if a.device != "cpu" and not a.stage_threads:
        a.stage_processes = True          # one interpreter (and one CUDA context) per stage, as a deployment runs them
    ov = {"tiny": True} if a.tiny else {}
    if a.thinker_layers:
        ov["thinker_layers"] = a.thinker_layers
    y = (YAML.replace("ASYNC_CHUNK", "true" if a.async_chunk else "false").replace("DEVICE", a.device)
         .replace("MAXB", str(a.max_concurrency)).replace("MAXTOK", str(a.max_tokens)).replace("CODEC", str(a.codec_frames))
         .replace("OVERRIDES", json.dumps(ov)).replace("THINKER_TP", str(a.thinker_tp))
         .replace("THINKER_EP", "true" if a.thinker_ep else "false")
         .replace("THINKER_DEVS", ",".join(str(i) for i in range(a.thinker_tp)))
         .replace("THINKER_PROC", "true" if (a.thinker_tp > 1 or a.stage_processes) else "false")
         .replace("STAGE_PROC", "true" if a.stage_processes else "false").replace("TAIL_DEV", str(a.tail_device)))
    f = tempfile.NamedTemporaryFile("w", suffix=".yaml", delete=False)
    f.write(y)
    f.close()
    return asyncio.run(_run(a, f.name))


if __name__ == "__main__":
    main()
