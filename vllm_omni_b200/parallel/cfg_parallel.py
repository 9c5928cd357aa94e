"""Classifier-free-guidance parallelism (degree 2).

Rank 0 of the CFG group runs the conditional branch, rank 1 the unconditional one.  The
reference all-gathers both predictions, mixes on rank 0, runs the scheduler there and
broadcasts the new latents (vllm_omni/diffusion/distributed/cfg_parallel.py:28-235: two NCCL
collectives plus several small kernels per step).  Here each rank publishes its prediction
in symmetric peer memory and ONE kernel per rank reads the partner's prediction over
NVLink, forms ``neg + s (pos - neg)``, applies the norm rescale and the flow-match Euler
update, so both ranks end the step with identical latents and nothing is broadcast.
Predictions are double-buffered by step parity; a bounded-wait device barrier per step orders
the exchange.  On CPU / Gloo the same result is produced with an all_gather (test path).
"""
from __future__ import annotations

import torch

from ..ops import fused


class CFGExchange:
    def __init__(self, group):
        if group.world_size != 2:
            raise ValueError("CFG parallel size must be 2")
        self.group = group
        self.rank = group.rank_in_group
        self.is_negative_rank = self.rank == 1
        self.arena = None
        self._key = None
        self._step = 0

    def _setup(self, v: torch.Tensor):
        key = (tuple(v.shape), v.dtype, str(v.device))
        if self._key == key:
            return
        self._key = key
        if self.arena is not None:
            self.arena.close()
        from .peer_memory import PeerArena
        self.arena = PeerArena(self.group, 2 * v.numel() * v.element_size() + 8192, v.device)
        self.slots = [self.arena.alloc(tuple(v.shape), v.dtype) for _ in range(2)]
        self._step = 0

    def step(self, v: torch.Tensor, latents: torch.Tensor, scale: float, dt: float, renorm: bool,
             lat_lowp: torch.Tensor | None = None):
        """v: this rank's velocity prediction; latents (fp32) updated in place on both ranks."""
        if not v.is_cuda:
            both = self.group.all_gather(v.contiguous(), separate_tensors=True)
            latents.copy_(fused.cfg_euler_step_reference(both[0], both[1], latents, scale, dt, renorm))
            if lat_lowp is not None:
                lat_lowp.copy_(latents)
            return latents
        self._setup(v)
        slot = self.slots[self._step & 1]
        self._step += 1
        slot.local.copy_(v)
        self.arena.barrier()
        mine, other = slot.ptrs[self.rank], slot.ptrs[1 - self.rank]
        pos, neg = (mine, other) if self.rank == 0 else (other, mine)
        fused.cfg_euler_step_(None, None, latents, scale, dt, renorm, lat_lowp, pos_ptr=pos, neg_ptr=neg)
        return latents

    def close(self):
        if self.arena is not None:
            self.arena.close()
            self.arena = None
