"""Serving benchmark client for an OpenAI-compatible omni server
(vllm_omni/benchmarks/patch/patch.py, benchmarks/diffusion/diffusion_benchmark_serving.py).

    python -m vllm_omni_b200.benchmarks.serve_bench serve --base-url http://127.0.0.1:8000 \
        --model Qwen/Qwen3-Omni-30B-A3B-Instruct --num-prompts 64 --max-concurrency 8 \
        --request-rate 4 --modalities text,audio
    python -m vllm_omni_b200.benchmarks.serve_bench image --base-url http://127.0.0.1:8000 \
        --model Qwen/Qwen-Image --num-prompts 16 --size 1024x1024 --num-inference-steps 50

``serve`` streams ``/v1/chat/completions`` and records time to first token, inter-token
latencies, time to first audio packet and the audio real-time factor; ``image`` posts to
``/v1/images/generations`` (or ``/v1/videos``) and records latency and throughput.  Arrivals are a
Poisson process at ``--request-rate`` (inf = all at once) under a concurrency cap.  The load
generator itself (``run_load``) takes any async request function, which is how the tests drive it
without a network.
"""
from __future__ import annotations

import argparse
import asyncio
import base64
import json
import random
import sys
import time
from typing import Awaitable, Callable

from .datasets import BenchRequest, random_multimodal_requests
from .metrics import RequestResult, summarize

RequestFn = Callable[[BenchRequest], Awaitable[RequestResult]]


async def run_load(request_fn: RequestFn, requests: list[BenchRequest], request_rate: float = float("inf"),
                   max_concurrency: int | None = None, seed: int = 0) -> tuple[list[RequestResult], float]:
    rng = random.Random(seed)
    sem = asyncio.Semaphore(max_concurrency) if max_concurrency else None
    results: list[RequestResult] = []

    async def one(r: BenchRequest):
        async def call():
            try:
                return await request_fn(r)
            except Exception as e:  # noqa: BLE001
                now = time.perf_counter()
                return RequestResult(ok=False, error=repr(e), start=now, end=now)
        if sem is None:
            results.append(await call())
        else:
            async with sem:
                results.append(await call())

    t0 = time.perf_counter()
    tasks = []
    for r in requests:
        tasks.append(asyncio.create_task(one(r)))
        if request_rate != float("inf") and request_rate > 0:
            await asyncio.sleep(rng.expovariate(request_rate))
    await asyncio.gather(*tasks)
    return results, time.perf_counter() - t0


def wav_seconds(b: bytes) -> float:
    """Duration of a PCM WAV blob (0 when the header is not understood)."""
    if len(b) < 44 or b[:4] != b"RIFF":
        return 0.0
    import struct
    ch, rate = struct.unpack("<HI", b[22:28])
    bits = struct.unpack("<H", b[34:36])[0]
    i = b.find(b"data")
    n = len(b) - (i + 8) if i >= 0 else 0
    return n / max(1, rate * ch * bits // 8)


def make_chat_request_fn(base_url: str, model: str, modalities=None, extra_body: dict | None = None,
                         timeout_s: float = 600.0) -> RequestFn:
    import aiohttp
    url = base_url.rstrip("/") + "/v1/chat/completions"

    async def fn(r: BenchRequest) -> RequestResult:
        body = {"model": model, "stream": True, "max_tokens": r.max_tokens,
                "messages": [{"role": "user", "content": r.content or r.prompt}]}
        if r.modalities or modalities:
            body["modalities"] = r.modalities or modalities
        body.update(extra_body or {})
        res = RequestResult(start=time.perf_counter(), prompt_tokens=r.prompt_len)
        last = res.start
        async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=timeout_s)) as sess:
            async with sess.post(url, json=body) as resp:
                if resp.status != 200:
                    res.ok, res.error = False, f"HTTP {resp.status}: {(await resp.text())[:200]}"
                    res.end = time.perf_counter()
                    return res
                async for raw in resp.content:
                    line = raw.decode().strip()
                    if not line.startswith("data:"):
                        continue
                    data = line[5:].strip()
                    if data == "[DONE]":
                        break
                    now = time.perf_counter()
                    ch = json.loads(data)
                    for c in ch.get("choices", []):
                        d = c.get("delta") or {}
                        if d.get("content"):
                            if res.ttft is None:
                                res.ttft = now - res.start
                            else:
                                res.itl.append(now - last)
                            last = now
                            res.output_tokens += 1
                        a = d.get("audio")
                        if a and a.get("data"):
                            if res.audio_ttfp is None:
                                res.audio_ttfp = now - res.start
                            res.audio_seconds += wav_seconds(base64.b64decode(a["data"]))
                    u = ch.get("usage")
                    if u:
                        res.output_tokens = u.get("completion_tokens", res.output_tokens)
                        res.prompt_tokens = u.get("prompt_tokens", res.prompt_tokens)
        res.end = time.perf_counter()
        return res

    return fn


def make_image_request_fn(base_url: str, model: str, size: str = "1024x1024", steps: int = 50, n: int = 1,
                          video: bool = False, extra_body: dict | None = None, timeout_s: float = 1800.0) -> RequestFn:
    import aiohttp
    url = base_url.rstrip("/") + ("/v1/videos" if video else "/v1/images/generations")

    async def fn(r: BenchRequest) -> RequestResult:
        body = {"model": model, "prompt": r.prompt, "size": size, "n": n, "num_inference_steps": steps,
                "response_format": "b64_json"}
        body.update(extra_body or {})
        res = RequestResult(start=time.perf_counter(), prompt_tokens=r.prompt_len)
        async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=timeout_s)) as sess:
            async with sess.post(url, json=body) as resp:
                txt = await resp.text()
                if resp.status != 200:
                    res.ok, res.error = False, f"HTTP {resp.status}: {txt[:200]}"
                else:
                    res.images = len(json.loads(txt).get("data", []))
        res.end = time.perf_counter()
        return res

    return fn


def main(argv=None) -> int:
    ap = argparse.ArgumentParser("serve_bench")
    ap.add_argument("what", choices=["serve", "image", "video"])
    ap.add_argument("--base-url", default="http://127.0.0.1:8000")
    ap.add_argument("--model", required=True)
    ap.add_argument("--num-prompts", type=int, default=32)
    ap.add_argument("--request-rate", type=float, default=float("inf"))
    ap.add_argument("--max-concurrency", type=int, default=None)
    ap.add_argument("--input-len", type=int, default=64)
    ap.add_argument("--output-len", type=int, default=64)
    ap.add_argument("--images-per-prompt", type=int, default=0)
    ap.add_argument("--audios-per-prompt", type=int, default=0)
    ap.add_argument("--modalities", default=None, help="comma list, e.g. text,audio")
    ap.add_argument("--size", default="1024x1024")
    ap.add_argument("--num-inference-steps", type=int, default=50)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--save-result", default=None)
    a = ap.parse_args(argv)
    mods = a.modalities.split(",") if a.modalities else None
    reqs = random_multimodal_requests(a.num_prompts, a.input_len, a.output_len, a.images_per_prompt,
                                      a.audios_per_prompt, seed=a.seed, modalities=mods)
    if a.what == "serve":
        fn = make_chat_request_fn(a.base_url, a.model, mods)
    else:
        fn = make_image_request_fn(a.base_url, a.model, a.size, a.num_inference_steps, video=a.what == "video")
    results, wall = asyncio.run(run_load(fn, reqs, a.request_rate, a.max_concurrency, a.seed))
    summary = summarize(results, wall)
    summary.update(model=a.model, what=a.what, num_prompts=a.num_prompts, request_rate=a.request_rate,
                   max_concurrency=a.max_concurrency)
    print(json.dumps(summary, indent=2))
    if a.save_result:
        with open(a.save_result, "w") as f:
            json.dump(summary, f)
    return 0 if summary["failed"] == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
