"""Thin wrappers around torch.distributed groups.

``GroupCoordinator`` owns a device group (NCCL on GPUs) and a CPU twin (Gloo) for one
family of rank groups and exposes the collectives the engine uses as the *baseline* path:
all_reduce, all_gather, gather, broadcast, object send/recv, tensor-dict broadcast
(vllm_omni/diffusion/distributed/group_coordinator.py:70-545).  The pipeline and
sequence-parallel variants add p2p helpers and the Ulysses / ring sub-groups (:548-938).
"""
from __future__ import annotations

import pickle
from typing import Any

import torch
import torch.distributed as dist


class GroupCoordinator:
    def __init__(self, group_ranks: list[list[int]], local_rank: int, backend: str, name: str = "group"):
        self.name = name
        self.rank = dist.get_rank()
        self.local_rank = local_rank
        self.device_group = None
        self.cpu_group = None
        self.ranks: list[int] = []
        for ranks in group_ranks:
            dg = dist.new_group(ranks, backend=backend)
            cg = dg if backend == "gloo" else dist.new_group(ranks, backend="gloo")
            if self.rank in ranks:
                self.ranks = list(ranks)
                self.device_group, self.cpu_group = dg, cg
        assert self.device_group is not None, f"rank {self.rank} is in no {name} group: {group_ranks}"
        self.world_size = len(self.ranks)
        self.rank_in_group = self.ranks.index(self.rank)
        self.device = torch.device("cuda", local_rank) if (backend == "nccl" and torch.cuda.is_available()) \
            else torch.device("cpu")

    # ranks -------------------------------------------------------------
    @property
    def first_rank(self): return self.ranks[0]
    @property
    def last_rank(self): return self.ranks[-1]
    @property
    def is_first_rank(self): return self.rank == self.first_rank
    @property
    def is_last_rank(self): return self.rank == self.last_rank
    @property
    def next_rank(self): return self.ranks[(self.rank_in_group + 1) % self.world_size]
    @property
    def prev_rank(self): return self.ranks[(self.rank_in_group - 1) % self.world_size]

    # collectives -------------------------------------------------------
    def all_reduce(self, x: torch.Tensor, op=dist.ReduceOp.SUM) -> torch.Tensor:
        if self.world_size == 1:
            return x
        dist.all_reduce(x, op=op, group=self.device_group)
        return x

    def all_gather(self, x: torch.Tensor, dim: int = 0, separate_tensors: bool = False):
        if self.world_size == 1:
            return [x] if separate_tensors else x
        x = x.contiguous()
        if x.dim() == 0:
            x = x.reshape(1)
        # the flat (concatenated along dim 0) form is the one both NCCL and Gloo accept
        flat = torch.empty((self.world_size * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(flat, x, group=self.device_group)
        out = flat.view((self.world_size,) + tuple(x.shape))
        if separate_tensors:
            return list(out.unbind(0))
        if dim < 0:
            dim += x.dim()
        out = out.movedim(0, dim)
        shape = list(x.shape)
        shape[dim] *= self.world_size
        return out.reshape(shape)

    def gather(self, x: torch.Tensor, dst: int = 0, dim: int = 0):
        """Gather to group-local rank ``dst``; other ranks get None."""
        if self.world_size == 1:
            return x
        lst = [torch.empty_like(x) for _ in range(self.world_size)] if self.rank_in_group == dst else None
        dist.gather(x.contiguous(), lst, dst=self.ranks[dst], group=self.device_group)
        return torch.cat(lst, dim=dim) if lst is not None else None

    def broadcast(self, x: torch.Tensor, src: int = 0) -> torch.Tensor:
        if self.world_size == 1:
            return x
        dist.broadcast(x, src=self.ranks[src], group=self.device_group)
        return x

    def reduce_scatter(self, x: torch.Tensor, dim: int = 0) -> torch.Tensor:
        if self.world_size == 1:
            return x
        xs = x.movedim(dim, 0).contiguous()
        out = torch.empty((xs.shape[0] // self.world_size,) + tuple(xs.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, xs, group=self.device_group)
        return out.movedim(0, dim)

    def all_to_all_single(self, out: torch.Tensor, inp: torch.Tensor):
        dist.all_to_all_single(out, inp, group=self.device_group)
        return out

    def barrier(self):
        if self.world_size > 1:
            dist.barrier(group=self.cpu_group)

    # objects on the CPU twin --------------------------------------------
    def broadcast_object(self, obj: Any = None, src: int = 0) -> Any:
        if self.world_size == 1:
            return obj
        lst = [obj]
        dist.broadcast_object_list(lst, src=self.ranks[src], group=self.cpu_group)
        return lst[0]

    def all_gather_object(self, obj: Any) -> list:
        if self.world_size == 1:
            return [obj]
        out = [None] * self.world_size
        dist.all_gather_object(out, obj, group=self.cpu_group)
        return out

    def send_object(self, obj: Any, dst: int) -> None:
        data = torch.frombuffer(bytearray(pickle.dumps(obj)), dtype=torch.uint8)
        size = torch.tensor([data.numel()], dtype=torch.long)
        dist.send(size, dst=self.ranks[dst], group=self.cpu_group)
        dist.send(data, dst=self.ranks[dst], group=self.cpu_group)

    def recv_object(self, src: int) -> Any:
        size = torch.empty(1, dtype=torch.long)
        dist.recv(size, src=self.ranks[src], group=self.cpu_group)
        data = torch.empty(int(size.item()), dtype=torch.uint8)
        dist.recv(data, src=self.ranks[src], group=self.cpu_group)
        return pickle.loads(data.numpy().tobytes())

    def broadcast_tensor_dict(self, d: dict | None = None, src: int = 0) -> dict:
        """Metadata (keys, shapes, dtypes, non-tensor values) over the CPU group, payloads
        over the device group."""
        if self.world_size == 1:
            return d
        if self.rank_in_group == src:
            meta = [(k, (tuple(v.shape), v.dtype, v.device.type) if isinstance(v, torch.Tensor) else ("obj", v))
                    for k, v in d.items()]
            self.broadcast_object(meta, src)
            for k, v in d.items():
                if isinstance(v, torch.Tensor) and v.numel():
                    grp = self.cpu_group if v.device.type == "cpu" else self.device_group
                    dist.broadcast(v.contiguous(), src=self.ranks[src], group=grp)
            return d
        meta = self.broadcast_object(None, src)
        out = {}
        for k, m in meta:
            if m[0] == "obj":
                out[k] = m[1]
                continue
            shape, dtype, devt = m
            t = torch.empty(shape, dtype=dtype, device=self.device if devt != "cpu" else "cpu")
            if t.numel():
                dist.broadcast(t, src=self.ranks[src], group=self.cpu_group if devt == "cpu" else self.device_group)
            out[k] = t
        return out

    def send_tensor_dict(self, d: dict, dst: int) -> None:
        meta = [(k, (tuple(v.shape), v.dtype) if isinstance(v, torch.Tensor) else ("obj", v)) for k, v in d.items()]
        self.send_object(meta, dst)
        for v in d.values():
            if isinstance(v, torch.Tensor) and v.numel():
                grp = self.cpu_group if v.device.type == "cpu" else self.device_group
                dist.send(v.contiguous(), dst=self.ranks[dst], group=grp)

    def recv_tensor_dict(self, src: int) -> dict:
        meta = self.recv_object(src)
        out = {}
        for k, m in meta:
            if m[0] == "obj":
                out[k] = m[1]
                continue
            t = torch.empty(m[0], dtype=m[1], device=self.device)
            if t.numel():
                grp = self.cpu_group if t.device.type == "cpu" else self.device_group
                dist.recv(t, src=self.ranks[src], group=grp)
            out[k] = t
        return out

    def destroy(self):
        for g in {self.device_group, self.cpu_group}:
            if g is not None:
                try:
                    dist.destroy_process_group(g)
                except Exception:
                    pass
        self.device_group = self.cpu_group = None


class PipelineGroupCoordinator(GroupCoordinator):
    """Adds stage-to-stage isend/irecv with shape exchange (PipeFusion-style patches)."""

    def pipeline_send(self, t: torch.Tensor, dst_offset: int = 1):
        dst = (self.rank_in_group + dst_offset) % self.world_size
        self.send_object((tuple(t.shape), t.dtype), dst)
        dist.send(t.contiguous(), dst=self.ranks[dst], group=self.device_group)

    def pipeline_recv(self, src_offset: int = -1) -> torch.Tensor:
        src = (self.rank_in_group + src_offset) % self.world_size
        shape, dtype = self.recv_object(src)
        t = torch.empty(shape, dtype=dtype, device=self.device)
        dist.recv(t, src=self.ranks[src], group=self.device_group)
        return t

    def pipeline_isend(self, t: torch.Tensor, dst_offset: int = 1):
        dst = (self.rank_in_group + dst_offset) % self.world_size
        return dist.isend(t.contiguous(), dst=self.ranks[dst], group=self.device_group)

    def pipeline_irecv(self, out: torch.Tensor, src_offset: int = -1):
        src = (self.rank_in_group + src_offset) % self.world_size
        return dist.irecv(out, src=self.ranks[src], group=self.device_group)


class SequenceParallelGroupCoordinator(GroupCoordinator):
    def __init__(self, group_ranks, local_rank, backend, ulysses_groups, ring_groups, name="sp"):
        super().__init__(group_ranks, local_rank, backend, name)
        self.ulysses = GroupCoordinator(ulysses_groups, local_rank, backend, name="ulysses")
        self.ring = GroupCoordinator(ring_groups, local_rank, backend, name="ring")

    @property
    def ulysses_group(self): return self.ulysses.device_group
    @property
    def ring_group(self): return self.ring.device_group
    @property
    def ulysses_world_size(self): return self.ulysses.world_size
    @property
    def ulysses_rank(self): return self.ulysses.rank_in_group
    @property
    def ring_world_size(self): return self.ring.world_size
    @property
    def ring_rank(self): return self.ring.rank_in_group

    def destroy(self):
        self.ulysses.destroy()
        self.ring.destroy()
        super().destroy()
