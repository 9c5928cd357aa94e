"""Spawn helper for multi-process tests (gloo on CPU, nccl on GPUs), rendezvous on 127.0.0.1."""
import os
import socket
import traceback

import torch
import torch.multiprocessing as mp


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, backend, args, errq):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), LOCAL_RANK=str(rank),
                      WORLD_SIZE=str(world))
    try:
        if backend == "nccl":
            torch.cuda.set_device(rank)
        fn(rank, world, *args)
    except Exception:
        errq.put((rank, traceback.format_exc()))
        raise
    finally:
        # a process group that is still alive when the interpreter tears down its threads can abort the process
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:   # noqa: BLE001
                pass


def run_distributed(fn, world: int, backend: str = "gloo", args=(), timeout: float = 240.0):
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, backend, args, errq)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.terminate()
    errs = []
    while not errq.empty():
        errs.append(errq.get())
    assert not alive, "distributed test timed out"
    assert not errs, "\n".join(f"[rank {r}]\n{tb}" for r, tb in errs)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
