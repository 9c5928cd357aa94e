"""Executors place diffusion workers on GPUs and run RPCs on them.

* ``UniProcExecutor``: the worker lives in the calling process.  With one GPU this is the
  lowest-latency path; under an external launcher (``torchrun``: one process per GPU, every
  process constructs the same engine) it is the SPMD path the scaling benchmark uses.
* ``MultiprocDiffusionExecutor``: spawns one ``worker_main`` process per GPU, ready
  handshake over pipes, RPC broadcast over per-worker queues, results from rank 0,
  liveness from ``is_alive`` plus a shared heartbeat counter
  (vllm_omni/diffusion/executor/multiproc_executor.py, abstract.py).
"""
from __future__ import annotations

import itertools
import multiprocessing as mp
import os
import time
from typing import Any

from ..logger import init_logger
from .data import OmniDiffusionConfig
from .worker import WorkerWrapperBase, worker_main

logger = init_logger(__name__)


class WorkerDeadError(RuntimeError):
    """A worker process exited or stopped heart-beating while a request was in flight."""


class DiffusionExecutor:
    def __init__(self, od_config: OmniDiffusionConfig):
        self.od_config = od_config

    def collective_rpc(self, method: str, args=(), kwargs=None, timeout: float | None = None,
                       output_rank: int = 0, unique_reply_rank: int | None = None) -> Any:
        raise NotImplementedError

    def add_req(self, req):
        return self.collective_rpc("generate", args=(req,))

    def check_health(self) -> bool:
        return True

    def shutdown(self):
        pass

    @staticmethod
    def get_class(od_config: OmniDiffusionConfig):
        backend = od_config.distributed_executor_backend
        external = int(os.environ.get("WORLD_SIZE", "1")) > 1 and "RANK" in os.environ
        if backend in ("uni", "external_launcher") or external or od_config.parallel_config.world_size == 1:
            return UniProcExecutor
        if backend == "mp":
            return MultiprocDiffusionExecutor
        raise ValueError(f"unknown distributed_executor_backend {backend!r}")


class UniProcExecutor(DiffusionExecutor):
    def __init__(self, od_config):
        super().__init__(od_config)
        external = int(os.environ.get("WORLD_SIZE", "1")) > 1 and "RANK" in os.environ
        rank = int(os.environ.get("RANK", "0")) if external else 0
        local_rank = int(os.environ.get("LOCAL_RANK", "0")) if external else 0
        if external and od_config.parallel_config.world_size != int(os.environ["WORLD_SIZE"]):
            raise ValueError(f"parallel_config world size {od_config.parallel_config.world_size} != WORLD_SIZE "
                             f"{os.environ['WORLD_SIZE']}")
        self.rank = rank
        self.worker = WorkerWrapperBase(local_rank, rank, od_config)
        self.worker.init_device(external_launcher=external)
        self.worker.load_model()

    def collective_rpc(self, method, args=(), kwargs=None, timeout=None, output_rank=0, unique_reply_rank=None):
        return getattr(self.worker, method)(*args, **(kwargs or {}))

    def shutdown(self):
        self.worker.shutdown()


class MultiprocDiffusionExecutor(DiffusionExecutor):
    HEARTBEAT_STALL_S = 120.0

    def __init__(self, od_config, init_timeout: float = 600.0, heartbeat_stall_s: float | None = None):
        super().__init__(od_config)
        self.heartbeat_stall_s = float(heartbeat_stall_s if heartbeat_stall_s is not None
                                       else os.environ.get("OMNI_WORKER_STALL_S", self.HEARTBEAT_STALL_S))
        ctx = mp.get_context("spawn")
        n = od_config.parallel_config.world_size
        self.res_q = ctx.Queue()
        self.cmd_qs, self.procs, self.heartbeats = [], [], []
        conns = []
        for r in range(n):
            cq = ctx.Queue()
            parent, child = ctx.Pipe(duplex=False)
            hb = ctx.Value("q", 0)
            p = ctx.Process(target=worker_main, args=(r, r, od_config, cq, self.res_q, child, hb), daemon=True,
                            name=f"omni-diffusion-worker-{r}")
            p.start()
            child.close()
            self.cmd_qs.append(cq); self.procs.append(p); self.heartbeats.append(hb); conns.append(parent)
        deadline = time.monotonic() + init_timeout
        for r, c in enumerate(conns):
            if not c.poll(max(0.0, deadline - time.monotonic())):
                self.shutdown()
                raise TimeoutError(f"diffusion worker {r} not ready after {init_timeout}s")
            msg = c.recv()
            if msg.get("status") != "ready":
                self.shutdown()
                raise RuntimeError(f"diffusion worker {r} failed to start: {msg.get('error')}")
        self._ids = itertools.count()

    def collective_rpc(self, method, args=(), kwargs=None, timeout=None, output_rank=0, unique_reply_rank=None):
        rid = next(self._ids)
        msg = {"type": "rpc", "id": rid, "method": method, "args": args, "kwargs": kwargs or {},
               "output_rank": output_rank, "exec_all_ranks": True}
        targets = range(len(self.cmd_qs)) if unique_reply_rank is None else [unique_reply_rank]
        for r in targets:
            self.cmd_qs[r].put(msg)
        deadline = None if timeout is None else time.monotonic() + timeout
        last_beats = [hb.value for hb in self.heartbeats]
        last_moved = [time.monotonic()] * len(last_beats)
        while True:
            try:
                res = self.res_q.get(timeout=0.2)
            except Exception:
                res = None
            if res is not None and res["id"] == rid:
                if res["error"]:
                    raise RuntimeError(f"worker rank {res['rank']} failed in {method}: {res['error']}")
                return res["result"]
            if not self.check_health():
                dead = [r for r, p in enumerate(self.procs) if not p.is_alive()]
                raise WorkerDeadError(f"diffusion worker(s) {dead} died during {method}")
            beats = [hb.value for hb in self.heartbeats]
            if beats != last_beats:
                moved = [r for r, (a, b) in enumerate(zip(beats, last_beats)) if a != b]
                for r in moved:
                    last_moved[r] = time.monotonic()
                last_beats = beats
            frozen = [r for r, t in enumerate(last_moved) if time.monotonic() - t > self.heartbeat_stall_s]
            if frozen:
                raise WorkerDeadError(f"diffusion worker(s) {frozen} stopped responding (no heartbeat for "
                                      f"{self.heartbeat_stall_s:.1f}s) during {method}")
            if deadline is not None and time.monotonic() > deadline:
                raise TimeoutError(f"collective_rpc({method}) timed out after {timeout}s")

    def check_health(self) -> bool:
        return all(p.is_alive() for p in self.procs)

    def shutdown(self):
        for q in self.cmd_qs:
            try:
                q.put({"type": "shutdown"})
            except Exception:
                pass
        for p in self.procs:
            p.join(timeout=5)
            if p.is_alive():
                p.terminate()
        self.cmd_qs, self.procs = [], []
