"""Baseline (library-collective) sequence-parallel communication.

``SeqAllToAll4D`` is the Ulysses head<->sequence exchange expressed with
``all_to_all_single`` and explicit layout copies, and ``RingComm`` the K/V ring shift with
batched isend/irecv — the mechanisms the reference uses
(vllm_omni/diffusion/distributed/comm.py:16-276).  They run on NCCL (GPU) and Gloo (CPU) and
serve as the measured baseline and the oracle for the fused kernels
(gemm scatter epilogue / attention scatter epilogue in csrc/).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def all_to_all_4d(x: torch.Tensor, scatter_idx: int, gather_idx: int, group=None) -> torch.Tensor:
    """x: [B, S, H, D].  (scatter 2, gather 1): [B, S/P, H, D] -> [B, S, H/P, D];
    (scatter 1, gather 2): [B, S, H/P, D] -> [B, S/P, H, D]."""
    P = dist.get_world_size(group)
    if P == 1:
        return x
    B, S, H, D = x.shape
    if scatter_idx == 2 and gather_idx == 1:
        assert H % P == 0
        t = x.reshape(B, S, P, H // P, D).permute(2, 0, 1, 3, 4).contiguous()     # [P, B, S, H/P, D]
        out = torch.empty_like(t)
        dist.all_to_all_single(out, t, group=group)
        return out.permute(1, 0, 2, 3, 4).reshape(B, P * S, H // P, D)
    if scatter_idx == 1 and gather_idx == 2:
        assert S % P == 0
        t = x.reshape(B, P, S // P, H, D).permute(1, 0, 2, 3, 4).contiguous()     # [P, B, S/P, H, D]
        out = torch.empty_like(t)
        dist.all_to_all_single(out, t, group=group)
        return out.permute(1, 2, 0, 3, 4).reshape(B, S // P, P * H, D)
    raise ValueError("scatter_idx / gather_idx must be (2, 1) or (1, 2)")


def all_to_all_5d(x: torch.Tensor, scatter_idx: int, gather_idx: int, group=None) -> torch.Tensor:
    """Packed qkv: [B, S, 3, H, D]; (scatter 3, gather 1) and its inverse (scatter 1, gather 3)."""
    B, S, T, H, D = x.shape
    if scatter_idx == 3 and gather_idx == 1:
        y = all_to_all_4d(x.permute(0, 1, 3, 2, 4).reshape(B, S, H, T * D), 2, 1, group)
        return y.reshape(B, y.shape[1], y.shape[2], T, D).permute(0, 1, 3, 2, 4)
    if scatter_idx == 1 and gather_idx == 3:
        y = all_to_all_4d(x.permute(0, 1, 3, 2, 4).reshape(B, S, H, T * D), 1, 2, group)
        return y.reshape(B, y.shape[1], y.shape[2], T, D).permute(0, 1, 3, 2, 4)
    raise ValueError("scatter_idx / gather_idx must be (3, 1) or (1, 3)")


class SeqAllToAll4D:
    @staticmethod
    def apply(group, x, scatter_idx: int = 2, gather_idx: int = 1):
        return all_to_all_4d(x, scatter_idx, gather_idx, group)


class SeqAllToAll5D:
    @staticmethod
    def apply(group, x, scatter_idx: int = 3, gather_idx: int = 1):
        return all_to_all_5d(x, scatter_idx, gather_idx, group)


class RingComm:
    """Ring neighbour exchange: ``send_recv`` posts the shift of a tensor to the next rank and
    the receive from the previous one; ``commit`` launches the batch, ``wait`` completes it."""

    def __init__(self, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        ranks = dist.get_process_group_ranks(group) if group is not None else list(range(self.world))
        self.send_rank = ranks[(self.rank + 1) % self.world]
        self.recv_rank = ranks[(self.rank - 1) % self.world]
        self._ops: list = []
        self._reqs = None

    def send_recv(self, to_send: torch.Tensor, recv_buf: torch.Tensor | None = None) -> torch.Tensor:
        res = recv_buf if recv_buf is not None else torch.empty_like(to_send)
        self._ops.append(dist.P2POp(dist.isend, to_send.contiguous(), self.send_rank, group=self.group))
        self._ops.append(dist.P2POp(dist.irecv, res, self.recv_rank, group=self.group))
        return res

    def commit(self):
        if self._reqs is not None:
            raise RuntimeError("commit called twice")
        self._reqs = dist.batch_isend_irecv(self._ops) if self._ops else []

    def wait(self):
        if self._reqs is None:
            raise RuntimeError("wait called before commit")
        for r in self._reqs:
            r.wait()
        self._reqs = None
        self._ops = []
