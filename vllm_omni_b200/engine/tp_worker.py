"""Tensor / expert parallel AR stages: one process per GPU, every rank runs the same engine.

The reference gets multi-GPU AR stages from vLLM's worker processes (vllm_omni/worker/gpu_ar_worker.py,
``tensor_parallel_size`` in vllm_omni/model_executor/stage_configs/qwen3_omni_moe.yaml:27): a
driver schedules and broadcasts the batch to the workers every step.  Here every rank of the
group owns a full ``LLMEngine`` (scheduler, paged-KV bookkeeping, runner) and the SAME request
stream, so the schedule is computed everywhere identically and nothing about the batch crosses
between processes; what crosses is
  * one small control message per step from rank 0 (requests added / aborted since the last
    step, or shutdown), over the group's Gloo twin,
  * the row-parallel partial sums inside the model (``parallel/tensor_parallel.RowParallelReduce``),
  * the sampled token ids of the step, broadcast from rank 0 on the device, so that a rounding
    difference between ranks can never split the request streams.
Rank 0 is the ``OmniLLM`` the stage runtime talks to; ranks 1.. are spawned by it and run
``follower_main``.
"""
from __future__ import annotations

import multiprocessing as mp
import os
import socket
import traceback

import torch


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class TPControl:
    """Control channel of the group: rank 0 sends one message per engine step."""

    def __init__(self, tp_group):
        self.group = tp_group
        self.rank, self.world = tp_group.rank_in_group, tp_group.world_size
        self.pending_add: list = []
        self.pending_abort: list = []

    def leader_step_message(self) -> None:
        msg = {"op": "step", "add": self.pending_add, "abort": self.pending_abort}
        self.pending_add, self.pending_abort = [], []
        self.group.broadcast_object(msg, src=0)

    def leader_shutdown(self) -> None:
        try:
            self.group.broadcast_object({"op": "shutdown"}, src=0)
        except Exception:   # noqa: BLE001  (followers already gone)
            pass

    def follower_recv(self) -> dict:
        return self.group.broadcast_object(None, src=0)


def init_tp_process(rank: int, world: int, port: int, use_cuda: bool, device_index: int, timeout_s: float = 600.0):
    """Join the stage's process group and build its tensor-parallel group."""
    from ..parallel import parallel_state as ps
    mine = {"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "RANK": str(rank), "WORLD_SIZE": str(world),
            "LOCAL_RANK": str(device_index)}
    saved = {k: os.environ.get(k) for k in mine}
    os.environ.update(mine)
    if use_cuda:
        torch.cuda.set_device(device_index)
    backend = "nccl" if use_cuda else "gloo"
    try:
        ps.init_distributed_environment(world_size=world, rank=rank, local_rank=device_index, backend=backend,
                                        timeout_s=timeout_s)
    finally:
        # the rendezvous variables are this stage's business only: rank 0 is the caller's own process, and
        # whatever it starts next (another stage, a diffusion executor) must not mistake itself for a rank
        for k, v in saved.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
    if not ps.model_parallel_is_initialized():
        ps.initialize_model_parallel(tensor_parallel_size=world, backend=backend)
    return ps.get_tp_group()


def follower_main(rank: int, world: int, port: int, model, kwargs: dict, device_index: int, ready, errq) -> None:
    """Entry point of ranks 1..: build the same stage engine, then mirror rank 0's steps."""
    try:
        from ..entrypoints.omni_llm import OmniLLM
        kw = dict(kwargs)
        kw["_tp_rank"], kw["_tp_port"], kw["_tp_device_index"] = rank, port, device_index
        llm = OmniLLM(model, **kw)
        ready.set()
        ctl = llm.tp_control
        while True:
            msg = ctl.follower_recv()
            if msg.get("op") == "shutdown":
                break
            for rid, prompt, sp in msg.get("add", ()):
                llm.engine.add_request(rid, prompt, sp)
            if msg.get("abort"):
                llm.engine.abort_request(msg["abort"])
            llm.engine.step()
    except BaseException as e:   # noqa: BLE001
        errq.put(f"rank {rank}: {type(e).__name__}: {e}\n{traceback.format_exc()}")
        ready.set()
        raise


def spawn_followers(world: int, port: int, model, kwargs: dict, device_indices: list[int]):
    """Start ranks 1..world-1; returns (processes, ready events, error queue)."""
    ctx = mp.get_context("spawn")
    errq = ctx.Queue()
    procs, readies = [], []
    for r in range(1, world):
        ev = ctx.Event()
        p = ctx.Process(target=follower_main, args=(r, world, port, model, kwargs, device_indices[r], ev, errq),
                        daemon=True, name=f"omni-tp-rank{r}")
        p.start()
        procs.append(p)
        readies.append(ev)
    return procs, readies, errq
