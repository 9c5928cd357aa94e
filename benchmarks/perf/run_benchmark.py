"""Performance regression gate (the reference's nightly ``tests/perf/scripts/run_benchmark.py`` +
``tests/perf/tests/test.json``): for every entry of a JSON file start a server, run the serving
benchmark over the entry's sweeps, and fail when a request did not complete or a metric exceeds
its baseline.

    python benchmarks/perf/run_benchmark.py --tests benchmarks/perf/tests.json --out perf_results.json
    python benchmarks/perf/run_benchmark.py --tests my.json --base-url http://127.0.0.1:8000     # server already up

Entry format:

    {"name": "qwen3_omni_text_audio",
     "server": {"model": "...", "args": ["--omni", "--stage-configs-path", "..."]},
     "kind": "serve" | "image",
     "sweeps": [{"num_prompts": 20, "request_rate": 0.5, "max_concurrency": 4, "input_len": 2500, "output_len": 900,
                 "modalities": ["text", "audio"]}],
     "baseline": {"mean_ttft_ms": 100000, "mean_audio_ttfp_ms": 100000, "mean_audio_rtf": 100000, "mean_e2el_ms": 1e9}}

Baselines are upper bounds (lower is better for all gated metrics).
"""
from __future__ import annotations

import argparse
import asyncio
import json
import os
import socket
import subprocess
import sys
import time
import urllib.request

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from vllm_omni_b200.benchmarks.datasets import random_multimodal_requests  # noqa: E402
from vllm_omni_b200.benchmarks.metrics import summarize  # noqa: E402
from vllm_omni_b200.benchmarks.serve_bench import make_chat_request_fn, make_image_request_fn, run_load  # noqa: E402

METRICS = {"mean_ttft_ms": ("ttft_s", "mean", 1e3), "p99_ttft_ms": ("ttft_s", "p99", 1e3),
           "mean_e2el_ms": ("e2el_s", "mean", 1e3), "mean_tpot_ms": ("tpot_s", "mean", 1e3),
           "mean_audio_ttfp_ms": ("audio_ttfp_s", "mean", 1e3), "mean_audio_rtf": ("audio_rtf", "mean", 1.0)}


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def start_server(model: str, args: list[str], timeout_s: float = 600.0):
    port = _free_port()
    cmd = [sys.executable, "-m", "vllm_omni_b200.entrypoints.cli.main", "serve", model, "--host", "127.0.0.1", "--port",
           str(port), *args]
    proc = subprocess.Popen(cmd, stdout=subprocess.DEVNULL, stderr=subprocess.STDOUT)
    url = f"http://127.0.0.1:{port}"
    t0 = time.monotonic()
    while time.monotonic() - t0 < timeout_s:
        if proc.poll() is not None:
            raise RuntimeError(f"server exited with code {proc.returncode}: {' '.join(cmd)}")
        try:
            with urllib.request.urlopen(url + "/health", timeout=1) as r:
                if r.status == 200:
                    return proc, url
        except OSError:
            time.sleep(0.5)
    proc.terminate()
    raise TimeoutError(f"server did not answer /health within {timeout_s:.0f} s")


def stop_server(proc) -> None:
    proc.terminate()
    try:
        proc.wait(timeout=20)
    except subprocess.TimeoutExpired:
        proc.kill()


def check(summary: dict, baseline: dict, num_prompts: int) -> list[str]:
    """Returns the list of violated gates (empty = pass)."""
    bad = []
    if summary["completed"] != num_prompts:
        bad.append(f"completed {summary['completed']} of {num_prompts} requests")
    for name, limit in (baseline or {}).items():
        if name not in METRICS:
            bad.append(f"unknown metric {name!r}")
            continue
        group, stat, scale = METRICS[name]
        v = (summary.get(group) or {}).get(stat)
        if v is None:
            continue                                   # metric not produced by this modality mix
        if v * scale > limit:
            bad.append(f"{name} = {v * scale:.3f} exceeds the baseline {limit}")
    return bad


def run_entry(entry: dict, base_url: str) -> list[dict]:
    model = entry["server"]["model"] if "server" in entry else entry.get("model", "model")
    out = []
    for sw in entry["sweeps"]:
        mods = sw.get("modalities")
        reqs = random_multimodal_requests(sw["num_prompts"], sw.get("input_len", 64), sw.get("output_len", 64),
                                          sw.get("images_per_prompt", 0), sw.get("audios_per_prompt", 0),
                                          seed=sw.get("seed", 0), modalities=mods)
        if entry.get("kind", "serve") == "serve":
            fn = make_chat_request_fn(base_url, model, mods, extra_body=sw.get("extra_body"))
        else:
            fn = make_image_request_fn(base_url, model, sw.get("size", "1024x1024"), sw.get("num_inference_steps", 50),
                                       video=entry.get("kind") == "video", extra_body=sw.get("extra_body"))
        results, wall = asyncio.run(run_load(fn, reqs, sw.get("request_rate", float("inf")), sw.get("max_concurrency"),
                                             sw.get("seed", 0)))
        summary = summarize(results, wall)
        out.append({"entry": entry["name"], "sweep": sw, "summary": summary,
                    "violations": check(summary, entry.get("baseline"), sw["num_prompts"])})
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser("perf-gate")
    ap.add_argument("--tests", required=True)
    ap.add_argument("--out", default=None)
    ap.add_argument("--base-url", default=None, help="use a running server instead of starting one per entry")
    ap.add_argument("--only", default=None, help="run the entry with this name only")
    a = ap.parse_args(argv)
    with open(a.tests) as f:
        entries = json.load(f)
    report = []
    for e in entries:
        if a.only and e["name"] != a.only:
            continue
        proc = None
        try:
            url = a.base_url
            if url is None:
                proc, url = start_server(e["server"]["model"], list(e["server"].get("args", [])),
                                         float(e["server"].get("startup_timeout_s", 600)))
            report.extend(run_entry(e, url))
        finally:
            if proc is not None:
                stop_server(proc)
    failed = [r for r in report if r["violations"]]
    for r in report:
        s = r["summary"]
        print(f"[{'FAIL' if r['violations'] else 'ok'}] {r['entry']} {r['sweep']}: completed {s['completed']}, "
              f"ttft {s['ttft_s'].get('mean', float('nan')) * 1e3:.1f} ms, e2e {s['e2el_s'].get('mean', float('nan')) * 1e3:.1f} ms"
              + "".join(f"\n      - {v}" for v in r["violations"]))
    if a.out:
        with open(a.out, "w") as f:
            json.dump(report, f, indent=1, default=str)
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
