"""Serving-benchmark metrics (vllm_omni/benchmarks/metrics/metrics.py): the usual request /
token latencies plus the audio ones — time to first audio packet (``audio_ttfp``) and the
real-time factor ``audio_rtf`` = generation time / seconds of audio produced."""
from __future__ import annotations

import statistics
from dataclasses import dataclass, field


@dataclass
class RequestResult:
    ok: bool = True
    error: str = ""
    start: float = 0.0
    end: float = 0.0
    ttft: float | None = None            # first text token
    audio_ttfp: float | None = None      # first audio packet
    itl: list[float] = field(default_factory=list)
    prompt_tokens: int = 0
    output_tokens: int = 0
    audio_seconds: float = 0.0
    images: int = 0
    video_frames: int = 0

    @property
    def latency(self) -> float:
        return self.end - self.start

    @property
    def audio_rtf(self) -> float | None:
        return self.latency / self.audio_seconds if self.audio_seconds > 0 else None


def _pct(xs, qs=(50, 90, 99)):
    xs = sorted(x for x in xs if x is not None)
    if not xs:
        return {}
    out = {"mean": statistics.fmean(xs)}
    for q in qs:
        out[f"p{q}"] = xs[min(len(xs) - 1, int(round(q / 100 * (len(xs) - 1))))]
    return out


def summarize(results: list[RequestResult], wall_s: float) -> dict:
    ok = [r for r in results if r.ok]
    out = {
        "completed": len(ok), "failed": len(results) - len(ok), "duration_s": wall_s,
        "request_throughput": len(ok) / wall_s if wall_s > 0 else 0.0,
        "output_token_throughput": sum(r.output_tokens for r in ok) / wall_s if wall_s > 0 else 0.0,
        "total_token_throughput": sum(r.output_tokens + r.prompt_tokens for r in ok) / wall_s if wall_s > 0 else 0.0,
        "image_throughput": sum(r.images for r in ok) / wall_s if wall_s > 0 else 0.0,
        "audio_seconds_per_s": sum(r.audio_seconds for r in ok) / wall_s if wall_s > 0 else 0.0,
        "e2el_s": _pct([r.latency for r in ok]),
        "ttft_s": _pct([r.ttft for r in ok]),
        "tpot_s": _pct([(r.latency - (r.ttft or 0.0)) / max(1, r.output_tokens - 1) for r in ok if r.output_tokens > 1]),
        "itl_s": _pct([x for r in ok for x in r.itl]),
        "audio_ttfp_s": _pct([r.audio_ttfp for r in ok]),
        "audio_rtf": _pct([r.audio_rtf for r in ok]),
    }
    return out
