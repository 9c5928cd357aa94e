"""Sequence-parallel self-attention for single-stream DiTs (Wan, Z-Image, FLUX single blocks ...).

The model keeps S / P rows of every sample on each rank; everything except self-attention is
row-local.  ``SequenceParallelAttention`` takes the local ``[B, S_loc, 3, H, Dh]`` q/k/v (already
normalised and rotated with the rows' own positions) and returns the local ``[B, S_loc, H, Dh]``
attention output over the FULL sequence:

* Ulysses degree U: head <-> sequence exchange inside the Ulysses group before and after; ``mode="peer"``:
  every rank publishes its rows in symmetric memory and pulls its heads of everybody's rows with the
  library's pitched copy kernel, and the attention kernel's epilogue stores each output row into the
  peer that owns it (two bounded barriers, no library collective); ``mode="nccl"``: all-to-all calls;
* ring degree R: the chunk's queries against every ring chunk's K/V — ``mode="peer"``: the other
  chunks are pulled once into a local buffer by this library's copy kernel on a side stream while
  the own chunk is attended to, and a second launch combines both results by their log-sum-exps in
  its epilogue; ``mode="nccl"``: send/recv around the ring with an eager merge (baseline, CPU);
* both: the hybrid grid of vllm_omni/diffusion/distributed/parallel_state.py:477-621.

``valid_len`` masks padding rows at the end of the global sequence (a model pads S up to a multiple
of P), the role of ``auto_pad`` in the reference's ``_sp_plan`` (sp_plan.py).
"""
from __future__ import annotations

import torch

from ..ops.attention import attention
from .comm import RingComm, all_to_all_4d, all_to_all_5d
from .ring import merge_attention


class SequenceParallelAttention:
    graph_safe = False

    def __init__(self, sp_group, num_heads: int, head_dim: int, mode: str | None = None):
        self.group = sp_group
        self.P, self.rank = sp_group.world_size, sp_group.rank_in_group
        self.U, self.R = sp_group.ulysses_world_size, sp_group.ring_world_size
        self.u, self.r = sp_group.ulysses_rank, sp_group.ring_rank
        if num_heads % self.U:
            raise ValueError(f"num_heads ({num_heads}) must be divisible by the Ulysses degree ({self.U})")
        self.H, self.Dh = num_heads, head_dim
        self.mode = mode or ("peer" if torch.cuda.is_available() else "nccl")
        self.arena = None
        self._key = None
        self._gath = self._own = self._side = None
        self._uly_arena = self._uly_key = None

    # rows ------------------------------------------------------------------------------
    def shard_rows(self, x: torch.Tensor, dim: int = 1):
        """Pad ``dim`` to a multiple of P with zeros and keep this rank's slice.  Returns
        (local slice, original length)."""
        S = x.shape[dim]
        pad = (-S) % self.P
        if pad:
            shape = list(x.shape)
            shape[dim] = pad
            x = torch.cat([x, x.new_zeros(shape)], dim=dim)
        per = x.shape[dim] // self.P
        return x.narrow(dim, self.rank * per, per).contiguous(), S

    def gather_rows(self, x: torch.Tensor, orig_len: int, dim: int = 1):
        return self.group.all_gather(x.contiguous(), dim=dim).narrow(dim, 0, orig_len)

    def local_rows(self, total_len: int) -> slice:
        per = (total_len + self.P - 1) // self.P
        return slice(self.rank * per, (self.rank + 1) * per)

    # attention -------------------------------------------------------------------------
    def _chunk_lens(self, valid_len, chunk, S_c, B, device):
        """Valid keys of ring chunk ``chunk``: ``valid_len`` is an int or an int tensor [B] of global
        lengths (everything past it, at the END of the global sequence, is padding)."""
        if valid_len is None:
            return None
        if torch.is_tensor(valid_len):
            return (valid_len.to(device) - chunk * S_c).clamp(0, S_c).to(torch.int32)
        n = max(0, min(S_c, int(valid_len) - chunk * S_c))
        return torch.full((B,), n, dtype=torch.int32, device=device)

    def _setup_arena(self, shape, dtype, device):
        key = (tuple(shape), dtype, str(device))
        if self._key == key:
            return
        self._key = key
        from .peer_memory import PeerArena
        if self.arena is not None:
            self.arena.close()
        n = 1
        for s in shape:
            n *= s
        self.arena = PeerArena(self.group.ring, n * torch.empty(0, dtype=dtype).element_size() + 8192, device)
        self.kv = self.arena.alloc(shape, dtype)

    # Ulysses exchange on own kernels ------------------------------------------------------
    def _uly_setup(self, B, S_loc, dtype, device):
        """Symmetric buffers of the Ulysses group: every rank publishes its [B, S_loc, 3, H, Dh] rows; the output
        rows of the attention come back through the kernel's scatter epilogue into [B, S_loc, H*Dh]."""
        key = (B, S_loc, dtype, str(device))
        if self._uly_key == key:
            return
        self._uly_key = key
        from .peer_memory import PeerArena
        if self._uly_arena is not None:
            self._uly_arena.close()
        es = torch.empty(0, dtype=dtype).element_size()
        HD = self.H * self.Dh
        self._uly_arena = PeerArena(self.group.ulysses, B * S_loc * 4 * HD * es + 16384, device)
        self._uly_pub = self._uly_arena.alloc((B, S_loc, 3, self.H, self.Dh), dtype)
        self._uly_out = self._uly_arena.alloc((B, S_loc, HD), dtype)
        Hu = self.H // self.U
        self._uly_joint = torch.empty(B, self.U * S_loc, 3, Hu, self.Dh, dtype=dtype, device=device)
        hoff = self.u * Hu * self.Dh * es
        self._uly_scatter = dict(n_peers=self.U, rows_per_rank=S_loc, rows_per_rank2=1, split=self.U * S_loc,
                                 o_ptrs=self._uly_out.peer_ptrs(hoff), o2_ptrs=self._uly_out.peer_ptrs(hoff),
                                 o_strides=(HD, self.Dh, S_loc * HD), o2_strides=(HD, self.Dh, S_loc * HD))

    def _uly_gather(self, q5):
        """Head <-> sequence exchange by pulls: this rank's H/U heads of q, k and v of every Ulysses peer's rows,
        one pitched copy per (peer, batch, q|k|v); rows end up ordered by source rank as an all-to-all leaves them."""
        from .peer_memory import pull_rows
        B, S_loc = q5.shape[0], q5.shape[1]
        self._uly_setup(B, S_loc, q5.dtype, q5.device)
        Hu, es = self.H // self.U, q5.element_size()
        seg = Hu * self.Dh
        self._uly_pub.local.copy_(q5)
        self._uly_arena.barrier()                         # every peer's rows are published
        j5 = self._uly_joint
        for p in range(self.U):
            for b in range(B):
                for w in range(3):
                    src = self._uly_pub.ptrs[p] + (((b * S_loc) * 3 + w) * self.H + self.u * Hu) * self.Dh * es
                    dst = j5[b, p * S_loc:(p + 1) * S_loc, w].reshape(S_loc, seg)      # a view: pitch 3 * seg elements
                    pull_rows(dst, src, 3 * self.H * self.Dh * es)
        return j5

    def __call__(self, q5: torch.Tensor, valid_len=None, scale: float | None = None) -> torch.Tensor:
        B, S_loc = q5.shape[0], q5.shape[1]
        uly_peer = self.U > 1 and self.mode == "peer" and q5.is_cuda
        sc = None
        if uly_peer:
            q5 = self._uly_gather(q5.contiguous())                                        # [B, S_c, 3, H/U, Dh]
            sc = self._uly_scatter                                                        # O rows go back to their owners
        elif self.U > 1:
            q5 = all_to_all_5d(q5.contiguous(), 3, 1, self.group.ulysses.device_group)    # [B, S_c, 3, H/U, Dh]
        S_c = q5.shape[1]
        q, k, v = q5[:, :, 0], q5[:, :, 1], q5[:, :, 2]
        dev = q5.device
        if self.R == 1:
            o = attention(q, k, v, kv_lens=self._chunk_lens(valid_len, 0, S_c, B, dev), scale=scale, scatter=sc)
        else:
            if valid_len is not None and int(torch.as_tensor(valid_len).min()) <= (self.R - 1) * S_c:
                raise ValueError("padding may not cover a whole ring chunk")
            out = lse = None
            if self.mode == "peer" and q5.is_cuda:
                # the other ring chunks' K/V are pulled once into a local buffer (side stream) while the own
                # chunk is attended to; the second launch combines both results in its epilogue
                from .peer_memory import pull_rows
                R, r = self.R, self.r
                Hu = q5.shape[3]
                shape = (B, S_c, 2, Hu, self.Dh)
                self._setup_arena(shape, q5.dtype, dev)
                self.kv.local.copy_(q5[:, :, 1:3])
                self.arena.barrier()
                chunk = S_c * 2 * Hu * self.Dh
                es = q5.element_size()
                from .ring import two_launches_pay
                overlap = two_launches_pay(B, S_c, Hu)
                srcs = [c for c in range(R) if c != r] if overlap else list(range(R))
                n = len(srcs)
                if self._gath is None or self._gath.shape != (B, n * chunk):
                    self._gath = torch.empty(B, n * chunk, dtype=q5.dtype, device=dev)
                    self._own = torch.empty(B, S_c, Hu, self.Dh, dtype=q5.dtype, device=dev)
                    self._side = self._side or torch.cuda.Stream(dev)
                main = torch.cuda.current_stream(dev)
                self._side.wait_stream(main)
                with torch.cuda.stream(self._side):
                    for j, src in enumerate(srcs):                         # one launch per chunk: a row per batch
                        if src != r:
                            pull_rows(self._gath[:, j * chunk:(j + 1) * chunk], self.kv.ptrs[src], chunk * es)
                g5 = self._gath.view(B, n * S_c, 2, Hu, self.Dh)
                if overlap:
                    # the own chunk in place while the pulls run, then the remote chunks with the combination
                    _, lse0 = attention(q, k, v, scale=scale, return_lse=True, out=self._own,
                                        kv_lens=self._chunk_lens(valid_len, r, S_c, B, dev))
                    main.wait_stream(self._side)
                    rem = None
                    if valid_len is not None:                               # padding sits at the end of the LAST chunk
                        rem = torch.stack([self._chunk_lens(valid_len, c, S_c, B, dev) for c in srcs]).sum(dim=0).to(torch.int32)
                    out = attention(q, g5[:, :, 0], g5[:, :, 1], scale=scale, kv_lens=rem, merge_prev=(self._own, lse0),
                                    out=self._own, scatter=sc)
                else:
                    # small grids: one launch over every chunk in order
                    pull_rows(self._gath[:, r * chunk:(r + 1) * chunk], self.kv.ptrs[r], chunk * es)
                    main.wait_stream(self._side)
                    lens = None
                    if valid_len is not None:
                        lens = (valid_len.to(dev) if torch.is_tensor(valid_len) else torch.full((B,), int(valid_len), device=dev)).to(torch.int32)
                    out = attention(q, g5[:, :, 0], g5[:, :, 1], scale=scale, kv_lens=lens, out=self._own, scatter=sc)
                self.arena.barrier()
            else:
                comm = RingComm(self.group.ring.device_group)
                k, v = k.contiguous(), v.contiguous()
                for step in range(self.R):
                    src = (self.r - step) % self.R
                    if step + 1 < self.R:
                        nk, nv_ = comm.send_recv(k), comm.send_recv(v)
                        comm.commit()
                    o_b, lse_b = attention(q, k, v, scale=scale, return_lse=True,
                                           kv_lens=self._chunk_lens(valid_len, src, S_c, B, dev))
                    out, lse = merge_attention(out, lse, o_b, lse_b)
                    if step + 1 < self.R:
                        comm.wait()
                        k, v = nk, nv_
            o = out.to(q5.dtype) if out is not None else None
        if uly_peer:
            self._uly_arena.barrier()                     # every owner has all heads of its rows
            return self._uly_out.local.view(B, S_loc, self.H, self.Dh)
        if self.U > 1:
            o = all_to_all_4d(o.contiguous(), 1, 2, self.group.ulysses.device_group)      # [B, S_loc, H, Dh]
        return o

    def close(self):
        if self._uly_arena is not None:
            self._uly_arena.close()
            self._uly_arena = None
        if self.arena is not None:
            self.arena.close()
            self.arena = None
