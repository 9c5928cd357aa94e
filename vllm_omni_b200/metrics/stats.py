"""Orchestrator-side statistics: per-stage request stats, inter-stage transfer edges and
end-to-end request records, with the summary tables ``--log-stats`` prints
(vllm_omni/metrics/stats.py:18-635; field glossary docs/contributing/metrics.md).
A Prometheus exposition (`render_prometheus`) is added for the `/metrics` route.
"""
from __future__ import annotations

import json
import time
from collections import defaultdict
from contextlib import contextmanager
from dataclasses import asdict, dataclass, field, fields
from typing import Any

from ..logger import init_logger

logger = init_logger(__name__)


@dataclass
class StageStats:
    total_token: int = 0
    total_gen_time_ms: float = 0.0

    @property
    def avg_tokens_per_s(self) -> float:
        return self.total_token * 1000.0 / self.total_gen_time_ms if self.total_gen_time_ms > 0 else 0.0


@dataclass
class StageRequestStats:
    batch_id: int = 0
    batch_size: int = 1
    num_tokens_in: int = 0
    num_tokens_out: int = 0
    stage_gen_time_ms: float = 0.0
    rx_transfer_bytes: int = 0
    rx_decode_time_ms: float = 0.0
    rx_in_flight_time_ms: float = 0.0
    stage_stats: StageStats | None = None
    stage_id: int | None = None
    final_output_type: str | None = None
    request_id: str | None = None
    postprocess_time_ms: float = 0.0
    diffusion_metrics: dict | None = None
    audio_generated_frames: int = 0

    @property
    def rx_mbps(self) -> float:
        if self.rx_transfer_bytes <= 0:
            return 0.0
        return float(self.rx_transfer_bytes) * 8.0 / (max(float(self.rx_decode_time_ms), 1e-6) * 1000.0)

    @property
    def tokens_per_s(self) -> float:
        return self.num_tokens_out * 1000.0 / self.stage_gen_time_ms if self.stage_gen_time_ms > 0 else 0.0


@dataclass
class TransferEdgeStats:
    from_stage: int
    to_stage: int
    request_id: str
    size_bytes: int = 0
    tx_time_ms: float = 0.0
    used_shm: bool = False
    rx_decode_time_ms: float = 0.0
    in_flight_time_ms: float = 0.0
    device_direct: bool = False      # payload went GPU->GPU without a host copy

    @property
    def total_time_ms(self) -> float:
        return float(self.tx_time_ms) + float(self.rx_decode_time_ms) + float(self.in_flight_time_ms)


@dataclass
class RequestE2EStats:
    request_id: str
    e2e_total_ms: float
    e2e_total_tokens: int
    transfers_total_time_ms: float
    transfers_total_bytes: int

    @property
    def e2e_tpt(self) -> float:
        return self.e2e_total_ms / self.e2e_total_tokens if self.e2e_total_tokens > 0 else 0.0


def format_table(title: str, rows: list[dict]) -> str:
    if not rows:
        return f"== {title}: (none) =="
    cols = list(rows[0].keys())
    def fmt(v):
        return f"{v:.3f}" if isinstance(v, float) else str(v)
    width = {c: max(len(c), *(len(fmt(r.get(c, ""))) for r in rows)) for c in cols}
    line = "+" + "+".join("-" * (width[c] + 2) for c in cols) + "+"
    out = [f"== {title} ==", line, "|" + "|".join(f" {c:<{width[c]}} " for c in cols) + "|", line]
    for r in rows:
        out.append("|" + "|".join(f" {fmt(r.get(c, '')):>{width[c]}} " for c in cols) + "|")
    out.append(line)
    return "\n".join(out)


class OrchestratorAggregator:
    def __init__(self, num_stages: int, log_stats: bool = False, log_file: str | None = None,
                 wall_start_ts: float | None = None):
        self.num_stages = num_stages
        self.log_stats = log_stats
        self.log_file = log_file
        self.init_run_state(wall_start_ts or time.time())

    def init_run_state(self, wall_start_ts: float) -> None:
        self.wall_start_ts = wall_start_ts
        self.stage_totals = [StageStats() for _ in range(self.num_stages)]
        self.stage_events: dict[str, list[StageRequestStats]] = defaultdict(list)
        self.transfer_events: dict[tuple, TransferEdgeStats] = {}
        self.e2e_events: list[RequestE2EStats] = []
        self.request_start: dict[str, float] = {}
        self.e2e_total_tokens = 0
        self.e2e_done = 0

    # ------------------------------------------------------------------ transfers
    def _edge(self, from_stage, to_stage, request_id) -> TransferEdgeStats:
        k = (from_stage, to_stage, request_id)
        if k not in self.transfer_events:
            self.transfer_events[k] = TransferEdgeStats(from_stage, to_stage, request_id)
        return self.transfer_events[k]

    def record_transfer_tx(self, from_stage, to_stage, request_id, size_bytes, tx_time_ms, used_shm=False,
                           device_direct=False):
        e = self._edge(from_stage, to_stage, request_id)
        e.size_bytes += int(size_bytes)
        e.tx_time_ms += float(tx_time_ms)
        e.used_shm = e.used_shm or used_shm
        e.device_direct = e.device_direct or device_direct
        return e

    def record_transfer_rx(self, from_stage, to_stage, request_id, rx_decode_time_ms, in_flight_time_ms=0.0):
        e = self._edge(from_stage, to_stage, request_id)
        e.rx_decode_time_ms += float(rx_decode_time_ms)
        e.in_flight_time_ms += float(in_flight_time_ms)
        return e

    # ------------------------------------------------------------------ stages
    def on_request_start(self, request_id: str, ts: float | None = None):
        self.request_start[request_id] = ts or time.time()

    def on_stage_metrics(self, stage_id: int, request_id: str, m: StageRequestStats | dict):
        if isinstance(m, dict):
            names = {f.name for f in fields(StageRequestStats)}
            m = StageRequestStats(**{k: v for k, v in m.items() if k in names})
        m.stage_id, m.request_id = stage_id, request_id
        tot = self.stage_totals[stage_id]
        tot.total_token += int(m.num_tokens_out)
        tot.total_gen_time_ms += float(m.stage_gen_time_ms)
        m.stage_stats = tot
        self.stage_events[request_id].append(m)

    def record_stage_postprocess_time(self, stage_id, request_id, ms):
        for ev in self.stage_events.get(request_id, []):
            if ev.stage_id == stage_id:
                ev.postprocess_time_ms += float(ms)

    @contextmanager
    def stage_postprocess_timer(self, stage_id, request_id):
        t = time.perf_counter()
        try:
            yield
        finally:
            self.record_stage_postprocess_time(stage_id, request_id, (time.perf_counter() - t) * 1e3)

    def record_audio_generated_frames(self, stage_id, request_id, frames: int):
        for ev in self.stage_events.get(request_id, []):
            if ev.stage_id == stage_id:
                ev.audio_generated_frames += int(frames)

    def on_finalize_request(self, request_id: str, ts: float | None = None) -> RequestE2EStats:
        t1 = ts or time.time()
        t0 = self.request_start.get(request_id, self.wall_start_ts)
        toks = sum(ev.num_tokens_out for ev in self.stage_events.get(request_id, []))
        edges = [e for (f, t, r), e in self.transfer_events.items() if r == request_id]
        ev = RequestE2EStats(request_id, (t1 - t0) * 1e3, toks, sum(e.total_time_ms for e in edges),
                             sum(e.size_bytes for e in edges))
        self.e2e_events.append(ev)
        self.e2e_total_tokens += toks
        self.e2e_done += 1
        return ev

    # ------------------------------------------------------------------ reports
    def build_summary(self, wall_s: float | None = None) -> dict[str, Any]:
        wall_ms = (wall_s if wall_s is not None else time.time() - self.wall_start_ts) * 1e3
        overall = {
            "e2e_requests": self.e2e_done, "e2e_wall_time_ms": wall_ms, "e2e_total_tokens": self.e2e_total_tokens,
            "e2e_avg_time_per_request_ms": wall_ms / self.e2e_done if self.e2e_done else 0.0,
            "e2e_avg_tokens_per_s": self.e2e_total_tokens * 1000.0 / wall_ms if wall_ms > 0 else 0.0,
        }
        for i, s in enumerate(self.stage_totals):
            overall[f"e2e_stage_{i}_wall_time_ms"] = s.total_gen_time_ms
        stages = []
        for rid, evs in self.stage_events.items():
            for ev in evs:
                stages.append({"request_id": rid, "stage_id": ev.stage_id, "batch_size": ev.batch_size,
                               "num_tokens_in": ev.num_tokens_in, "num_tokens_out": ev.num_tokens_out,
                               "stage_gen_time_ms": ev.stage_gen_time_ms, "tokens_per_s": ev.tokens_per_s,
                               "postprocess_time_ms": ev.postprocess_time_ms,
                               "audio_generated_frames": ev.audio_generated_frames})
        transfers = [{"edge": f"{e.from_stage}->{e.to_stage}", "request_id": e.request_id,
                      "size_kbytes": e.size_bytes / 1024.0, "tx_time_ms": e.tx_time_ms,
                      "rx_decode_time_ms": e.rx_decode_time_ms, "in_flight_time_ms": e.in_flight_time_ms,
                      "device_direct": e.device_direct} for e in self.transfer_events.values()]
        e2e = [{"request_id": e.request_id, "e2e_total_ms": e.e2e_total_ms, "e2e_total_tokens": e.e2e_total_tokens,
                "e2e_tpt": e.e2e_tpt, "transfers_total_time_ms": e.transfers_total_time_ms,
                "transfers_total_kbytes": e.transfers_total_bytes / 1024.0} for e in self.e2e_events]
        return {"overall": overall, "stages": stages, "transfers": transfers, "e2e": e2e}

    def build_and_log_summary(self, wall_s: float | None = None) -> dict[str, Any]:
        s = self.build_summary(wall_s)
        if self.log_stats:
            text = "\n".join([format_table("overall", [s["overall"]]), format_table("stages", s["stages"]),
                              format_table("transfers", s["transfers"]), format_table("requests", s["e2e"])])
            print(text, flush=True)
        if self.log_file:
            with open(self.log_file, "a") as f:
                f.write(json.dumps(s) + "\n")
        return s

    def render_prometheus(self) -> str:
        s = self.build_summary()
        out = ["# TYPE omni_e2e_requests counter", f"omni_e2e_requests {s['overall']['e2e_requests']}",
               "# TYPE omni_e2e_tokens counter", f"omni_e2e_tokens {s['overall']['e2e_total_tokens']}"]
        for i, st in enumerate(self.stage_totals):
            out.append(f'omni_stage_gen_time_ms{{stage="{i}"}} {st.total_gen_time_ms}')
            out.append(f'omni_stage_tokens{{stage="{i}"}} {st.total_token}')
        tx = defaultdict(lambda: [0, 0.0])
        for e in self.transfer_events.values():
            k = f"{e.from_stage}->{e.to_stage}"
            tx[k][0] += e.size_bytes
            tx[k][1] += e.total_time_ms
        for k, (b, ms) in tx.items():
            out.append(f'omni_transfer_bytes{{edge="{k}"}} {b}')
            out.append(f'omni_transfer_time_ms{{edge="{k}"}} {ms}')
        return "\n".join(out) + "\n"
