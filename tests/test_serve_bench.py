"""Serving benchmark client: the load generator with a scripted request function, the WAV
duration parser, and the HTTP image path against a real (uvicorn) server with a fake engine."""
import asyncio
import socket
import threading
import time

import pytest

from vllm_omni_b200.benchmarks.datasets import random_multimodal_requests
from vllm_omni_b200.benchmarks.metrics import RequestResult, summarize
from vllm_omni_b200.benchmarks.serve_bench import make_image_request_fn, run_load, wav_seconds


def test_run_load_concurrency_cap_and_summary():
    reqs = random_multimodal_requests(12, input_len=8, output_len=4, images=1, audios=1, seed=3)
    assert len(reqs[0].content) == 3 and reqs[0].content[1]["type"] == "image_url"
    live, peak = 0, 0

    async def fn(r):
        nonlocal live, peak
        live += 1
        peak = max(peak, live)
        t0 = time.perf_counter()
        await asyncio.sleep(0.01)
        live -= 1
        if r is reqs[5]:
            raise RuntimeError("boom")
        return RequestResult(start=t0, end=time.perf_counter(), ttft=0.004, itl=[0.002, 0.003], prompt_tokens=8,
                             output_tokens=4, audio_ttfp=0.006, audio_seconds=0.5)

    results, wall = asyncio.run(run_load(fn, reqs, request_rate=2000.0, max_concurrency=3))
    assert peak <= 3 and len(results) == 12
    s = summarize(results, wall)
    assert s["completed"] == 11 and s["failed"] == 1
    assert s["audio_ttfp_s"]["p50"] == 0.006 and s["audio_rtf"]["mean"] > 0
    assert s["output_token_throughput"] == pytest.approx(44 / wall)


def test_wav_seconds():
    from vllm_omni_b200.benchmarks.datasets import _wav_b64
    import base64
    import random
    assert wav_seconds(base64.b64decode(_wav_b64(random.Random(0), 0.25))) == pytest.approx(0.25, abs=1e-3)
    assert wav_seconds(b"nope") == 0.0


def test_image_bench_over_http():
    uvicorn = pytest.importorskip("uvicorn")
    from test_openai_api import FakeDiffusionEngine
    from vllm_omni_b200.entrypoints.openai.api_server import build_app
    app = build_app(FakeDiffusionEngine(), "fake", kind="diffusion")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="error"))
    th = threading.Thread(target=server.run, daemon=True)
    th.start()
    try:
        for _ in range(100):
            if server.started:
                break
            time.sleep(0.05)
        assert server.started
        fn = make_image_request_fn(f"http://127.0.0.1:{port}", "fake", size="32x32", steps=2)
        reqs = random_multimodal_requests(4, input_len=5, seed=1)
        results, wall = asyncio.run(run_load(fn, reqs, max_concurrency=2))
        s = summarize(results, wall)
        assert s["completed"] == 4 and s["failed"] == 0 and s["image_throughput"] > 0
    finally:
        server.should_exit = True
        th.join(timeout=5)


def test_perf_gate_passes_and_fails_on_baselines(tmp_path):
    """The regression gate against a live (fake-engine) server: every request must complete and the
    gated metrics must stay under their baselines."""
    uvicorn = pytest.importorskip("uvicorn")
    import importlib.util
    import json
    import os
    from test_openai_api import FakeDiffusionEngine
    from vllm_omni_b200.entrypoints.openai.api_server import build_app
    spec = importlib.util.spec_from_file_location(
        "perf_gate", os.path.join(os.path.dirname(__file__), "..", "benchmarks", "perf", "run_benchmark.py"))
    gate = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gate)
    app = build_app(FakeDiffusionEngine(), "fake", kind="diffusion")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="error"))
    th = threading.Thread(target=server.run, daemon=True)
    th.start()
    try:
        for _ in range(100):
            if server.started:
                break
            time.sleep(0.05)
        entry = {"name": "img", "kind": "image", "model": "fake",
                 "sweeps": [{"num_prompts": 3, "max_concurrency": 2, "size": "32x32", "num_inference_steps": 2}]}
        tests = tmp_path / "t.json"
        tests.write_text(json.dumps([dict(entry, baseline={"mean_e2el_ms": 60000})]))
        out = tmp_path / "r.json"
        assert gate.main(["--tests", str(tests), "--base-url", f"http://127.0.0.1:{port}", "--out", str(out)]) == 0
        rep = json.loads(out.read_text())
        assert rep[0]["summary"]["completed"] == 3 and rep[0]["violations"] == []
        tests.write_text(json.dumps([dict(entry, baseline={"mean_e2el_ms": 1e-6})]))
        assert gate.main(["--tests", str(tests), "--base-url", f"http://127.0.0.1:{port}"]) == 1
    finally:
        server.should_exit = True
        th.join(timeout=5)
    # the shipped gate file is well formed
    shipped = json.load(open(os.path.join(os.path.dirname(__file__), "..", "benchmarks", "perf", "tests.json")))
    assert all(set(e["baseline"]) <= set(gate.METRICS) and e["sweeps"] for e in shipped)
    assert gate.check({"completed": 2, "ttft_s": {"mean": 0.5}}, {"mean_ttft_ms": 400}, 3) == [
        "completed 2 of 3 requests", "mean_ttft_ms = 500.000 exceeds the baseline 400"]
