"""Hybrid Ulysses x ring sequence parallelism (P5).

The SP group of U * R ranks is a grid: ``ulysses`` groups are the contiguous runs of U ranks (one
ring chunk of the sequence each), ``ring`` groups connect the ranks with the same position in
their run (vllm_omni/diffusion/distributed/parallel_state.py:477-621).  Rank (u, r) owns
S / (U R) rows.  Per block:

1. head <-> sequence all-to-all INSIDE the Ulysses group (the fused GEMM-epilogue scatter on
   GPUs): the rank now holds q, k, v of ring chunk r (S / R rows) for its H / U heads;
2. attention of that chunk's queries against the keys of EVERY ring chunk: the R ranks of the ring
   group publish their K/V in symmetric memory; a side stream pulls the other chunks into one
   local buffer with this library's copy kernel (each remote byte crosses NVLink once) while the
   main stream attends to the own chunk; a second launch attends to the gathered chunks and
   combines both results by their log-sum-exps in its epilogue;
3. that same epilogue stores every output row into the Ulysses peer that owns it (the reverse
   all-to-all), so the local rows have all heads again after one barrier.

``mode="nccl"`` does steps 1-3 with collectives and send/recv (baseline and CPU test path).
"""
from __future__ import annotations

import torch

from ..ops.attention import attention
from .comm import RingComm, all_to_all_4d
from .ring import merge_attention
from .ulysses import UlyssesJointAttention


class HybridJointAttention:
    graph_safe = False        # the NCCL baseline mode is not capturable; the peer mode would be

    def __init__(self, sp_group, num_heads: int, head_dim: int, mode: str | None = None):
        self.group = sp_group
        self.P, self.rank = sp_group.world_size, sp_group.rank_in_group
        self.U, self.R = sp_group.ulysses_world_size, sp_group.ring_world_size
        self.u, self.r = sp_group.ulysses_rank, sp_group.ring_rank
        if self.rank != self.r * self.U + self.u:
            raise ValueError("the SP group must be laid out with Ulysses ranks contiguous")
        self.mode = mode or ("peer" if torch.cuda.is_available() else "nccl")
        self.uly = UlyssesJointAttention(sp_group.ulysses, num_heads, head_dim,
                                         mode="fused" if self.mode == "peer" else "nccl")
        self.uly.use_flags = False       # this class orders its exchanges with barriers and NCCL calls
        self.H, self.Dh, self.Hp = num_heads, head_dim, num_heads // self.U
        self.arena = None
        self._key = None
        self._side = self._gath = self._overlap = None

    def setup(self, B, Si_loc, St_loc, device, dtype):
        self.uly.setup(B, Si_loc, St_loc, device, dtype)
        key = (B, Si_loc, St_loc, str(device), dtype)
        if self._key == key:
            return
        self._key = key
        self._side = self._gath = None
        self.B, self.Si_loc, self.St_loc = B, Si_loc, St_loc
        self.Si_c, self.St_c = Si_loc * self.U, St_loc * self.U          # rows of one ring chunk
        self.S_c = self.Si_c + self.St_c
        self.S_img, self.S_txt = self.Si_c * self.R, self.St_c * self.R
        if self.mode == "peer":
            from .peer_memory import PeerArena
            if self.arena is not None:
                self.arena.close()
            es = torch.empty(0, dtype=dtype).element_size()
            self.arena = PeerArena(self.group.ring, B * self.S_c * 2 * self.Hp * self.Dh * es + 8192, device)
            self.kv = self.arena.alloc((B, self.S_c, 2, self.Hp, self.Dh), dtype)

    # same interface as UlyssesJointAttention -------------------------------------------
    def project_qkv(self, img_lin, xn_img, txt_lin, xn_txt):
        self.uly.project_qkv(img_lin, xn_img, txt_lin, xn_txt)

    def norm_rope(self, wq, wk, wq_txt, wk_txt, cos, sin, eps):
        # this chunk's rows of the global [all image rows, all text rows] position table
        r = self.r
        idx = torch.cat([torch.arange(r * self.Si_c, (r + 1) * self.Si_c),
                         torch.arange(self.S_img + r * self.St_c, self.S_img + (r + 1) * self.St_c)]).to(cos.device)
        self.uly.norm_rope(wq, wk, wq_txt, wk_txt, cos[idx].contiguous(), sin[idx].contiguous(), eps)

    def _chunk_kv_lens(self, kv_lens, chunk):
        if kv_lens is None:
            return None
        txt_valid = (kv_lens - self.S_img - chunk * self.St_c).clamp(0, self.St_c)
        return (self.Si_c + txt_valid).to(torch.int32)

    def attend(self, kv_lens, ws):
        B = self.B
        q5 = self.uly.joint_local.view(B, self.S_c, 3, self.Hp, self.Dh)
        q = q5[:, :, 0]
        out = lse = None
        if self.mode == "peer":
            from .peer_memory import pull_rows
            R, r, Sc = self.R, self.r, self.S_c
            dev = q.device
            self.kv.local.copy_(q5[:, :, 1:3])
            self.arena.barrier()                                  # every chunk's K/V is published
            sc = self.uly._attn_scatter                           # rows go to their owner inside the Ulysses group
            if R == 1:
                attention(q, q5[:, :, 1], q5[:, :, 2], kv_lens=self._chunk_kv_lens(kv_lens, r), scatter=sc)
            else:
                from .ring import two_launches_pay
                main = torch.cuda.current_stream(dev)
                overlap = two_launches_pay(B, Sc, self.Hp)
                if self._side is None or self._overlap != overlap:
                    self._side, self._overlap = torch.cuda.Stream(dev), overlap
                    # chunks in ring order (image rows, then text rows: valid keys stay a prefix); the overlapped
                    # form leaves the own chunk out of the buffer and reads it in place
                    self._srcs = [c for c in range(R) if c != r] if overlap else list(range(R))
                    self._gath = torch.empty(B, len(self._srcs) * Sc, 2 * self.Hp * self.Dh, dtype=q.dtype, device=dev)
                    self._own = torch.empty(B, Sc, self.Hp, self.Dh, dtype=q.dtype, device=dev)
                    self._srcs_t = torch.tensor(self._srcs, device=dev, dtype=torch.int32)
                n = len(self._srcs)
                row = 2 * self.Hp * self.Dh
                es = q.element_size()

                def pull(j, src):
                    for b in range(B):
                        base = self.kv.ptrs[src] + b * Sc * row * es
                        pull_rows(self._gath[b, j * self.Si_c:(j + 1) * self.Si_c], base, row * es)
                        if self.St_c:
                            t0 = n * self.Si_c + j * self.St_c
                            pull_rows(self._gath[b, t0:t0 + self.St_c], base + self.Si_c * row * es, row * es)
                self._side.wait_stream(main)
                with torch.cuda.stream(self._side):
                    for j, src in enumerate(self._srcs):
                        if src != r:
                            pull(j, src)
                g5 = self._gath.view(B, n * Sc, 2, self.Hp, self.Dh)
                if overlap:
                    _, lse0 = attention(q, q5[:, :, 1], q5[:, :, 2], kv_lens=self._chunk_kv_lens(kv_lens, r), return_lse=True,
                                        out=self._own)
                    main.wait_stream(self._side)
                    rem = None
                    if kv_lens is not None:
                        txt = (kv_lens[:, None] - self.S_img - self._srcs_t[None] * self.St_c).clamp(0, self.St_c).sum(dim=1)
                        rem = (n * self.Si_c + txt).to(torch.int32)
                    attention(q, g5[:, :, 0], g5[:, :, 1], kv_lens=rem, merge_prev=(self._own, lse0), scatter=sc)
                else:
                    pull(r, r)
                    main.wait_stream(self._side)
                    attention(q, g5[:, :, 0], g5[:, :, 1], kv_lens=kv_lens.to(torch.int32) if kv_lens is not None else None,
                              scatter=sc)
            self.arena.barrier()                                  # published K/V may be overwritten
            self.uly.arena.barrier()                              # every owner has its rows
            return self.uly.attn_img.local, self.uly.attn_txt.local
        else:
            comm = RingComm(self.group.ring.device_group)
            k, v = q5[:, :, 1].contiguous(), q5[:, :, 2].contiguous()
            for step in range(self.R):
                src = (self.r - step) % self.R
                if step + 1 < self.R:
                    nk, nv_ = comm.send_recv(k), comm.send_recv(v)
                    comm.commit()
                o_b, lse_b = attention(q, k, v, kv_lens=self._chunk_kv_lens(kv_lens, src), return_lse=True)
                out, lse = merge_attention(out, lse, o_b, lse_b)
                if step + 1 < self.R:
                    comm.wait()
                    k, v = nk, nv_
        o = out.to(q.dtype)                                       # [B, S_c, Hp, Dh]
        grp = self.group.ulysses.device_group
        oi = all_to_all_4d(o[:, :self.Si_c].contiguous(), 1, 2, grp).reshape(B, self.Si_loc, self.H * self.Dh)
        ot = None
        if self.St_loc:
            ot = all_to_all_4d(o[:, self.Si_c:].contiguous(), 1, 2, grp).reshape(B, self.St_loc, self.H * self.Dh)
        return oi, ot

    def close(self):
        self.uly.close()
        if self.arena is not None:
            self.arena.close()
            self.arena = None
