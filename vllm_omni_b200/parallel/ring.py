"""Ring / peer-KV attention for sequence parallelism (K5).

Each rank owns S/P rows (image and text sharded alike) and ALL heads.  Attention over the full
sequence = merge of P partial attentions, one per K/V shard:
    out = out - sigmoid(lse_b - lse) * (out - out_b),   lse = lse - logsigmoid(lse - lse_b)
(the update rule of vllm_omni/diffusion/attention/backends/ring/ring_utils.py:79-80).

``mode="peer"`` (GPU): every rank publishes its K/V shard in symmetric peer memory once per
layer; behind NVSwitch there is no ring to walk.  A side stream pulls the K/V of ALL other ranks
into one local buffer with this library's copy kernel (each remote byte crosses NVLink once;
reading the peer's tiles straight from the attention kernel makes every query-tile CTA fetch them
again: 354 us against 107 us with local K/V at 2048 rows x 24 heads on two B200s).  Small grids
then run ONE launch over all keys in global order; grids that fill the GPU several times over
attend to the own shard while the pulls run and finish with a second launch whose epilogue combines
both results by their log-sum-exps (``attention(..., merge_prev=...)``).  Either way at most two
launches per layer whatever the degree, and no merge kernels.  One bounded-wait barrier before
(shards written) and one after (shards consumed) per layer.
``mode="nccl"``: classic ring with batched isend/irecv of K and V (the baseline; also the CPU
test path).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..ops import fused
from ..ops.attention import attention
from .comm import RingComm


def two_launches_pay(B: int, S_q: int, H: int) -> bool:
    """Whether the ring's "own shard while the remote ones are pulled, then the rest" form beats one
    launch over all gathered keys: only when a launch fills the GPU several times over, so that cutting
    the key set in two does not leave both launches with a ragged last wave.  ``OMNI_RING_MODE`` =
    ``overlap`` / ``single`` forces either."""
    import os
    mode = os.environ.get("OMNI_RING_MODE")
    if mode in ("overlap", "single"):
        return mode == "overlap"
    return B * H * -(-S_q // 256) >= 4 * 148


def merge_attention(out, lse, out_b, lse_b):
    """Numerically stable merge of two partial attentions.  out: [B,S,H,D] fp32, lse: [B,H,S]."""
    if out is None:
        return out_b.float(), lse_b
    l, lb = lse.transpose(1, 2).unsqueeze(-1), lse_b.transpose(1, 2).unsqueeze(-1)     # [B,S,H,1]
    new_out = out - torch.sigmoid(lb - l) * (out - out_b.float())
    new_lse = lse - F.logsigmoid(lse - lse_b)
    return new_out, new_lse


class RingJointAttention:
    def __init__(self, group, num_heads: int, head_dim: int, mode: str | None = None):
        self.group = group
        self.P, self.rank = group.world_size, group.rank_in_group
        self.H, self.Dh = num_heads, head_dim
        self.mode = mode or ("peer" if torch.cuda.is_available() else "nccl")
        self.arena = None
        self._key = None
        self._side = self._gath = self._overlap = None

    def setup(self, B, Si_loc, St_loc, device, dtype):
        key = (B, Si_loc, St_loc, str(device), dtype)
        if self._key == key:
            return
        self._key = key
        self._side = self._gath = None
        self.B, self.Si_loc, self.St_loc = B, Si_loc, St_loc
        self.S_loc = Si_loc + St_loc
        self.S_img, self.S_txt = Si_loc * self.P, St_loc * self.P
        HD = self.H * self.Dh
        if self.mode == "peer":
            from .peer_memory import PeerArena
            if self.arena is not None:
                self.arena.close()
            es = torch.empty(0, dtype=dtype).element_size()
            self.arena = PeerArena(self.group, B * self.S_loc * 3 * HD * es + 8192, device)
            self.qkv = self.arena.alloc((B, self.S_loc, 3 * HD), dtype)
            self.qkv_local = self.qkv.local
        else:
            self.qkv_local = torch.empty(B, self.S_loc, 3 * HD, dtype=dtype, device=device)
        self.attn = torch.empty(B, self.S_loc, HD, dtype=dtype, device=device)

    # same interface as UlyssesJointAttention --------------------------------------------
    def project_qkv(self, img_lin, xn_img, txt_lin, xn_txt):
        HD, B = self.H * self.Dh, self.B
        bs = self.S_loc * 3 * HD
        img_lin(xn_img, out=self.qkv_local[:, :self.Si_loc], out_rows_per_batch=self.Si_loc, out_batch_stride=bs)
        if self.St_loc:
            txt_lin(xn_txt, out=self.qkv_local[:, self.Si_loc:], out_rows_per_batch=self.St_loc, out_batch_stride=bs)

    def norm_rope(self, wq, wk, wq_txt, wk_txt, cos, sin, eps):
        # local rows: image rows r*Si_loc.., text rows S_img + r*St_loc.. of the global table
        r = self.rank
        idx = torch.cat([torch.arange(r * self.Si_loc, (r + 1) * self.Si_loc),
                         torch.arange(self.S_img + r * self.St_loc, self.S_img + (r + 1) * self.St_loc)]).to(cos.device)
        fused.qk_norm_rope_(self.qkv_local, self.H, self.H, self.Dh, wq=wq, wk=wk, wq_alt=wq_txt, wk_alt=wk_txt,
                            s_alt=self.Si_loc, cos=cos[idx].contiguous(), sin=sin[idx].contiguous(), interleaved=True,
                            eps=eps)

    def _shard_kv_lens(self, kv_lens, src_rank):
        """Valid keys inside the shard of ``src_rank``: all image rows, text rows below the length."""
        if kv_lens is None:
            return None
        txt_valid = (kv_lens - self.S_img - src_rank * self.St_loc).clamp(0, self.St_loc)
        return (self.Si_loc + txt_valid).to(torch.int32)

    def attend(self, kv_lens, ws):
        B, HD = self.B, self.H * self.Dh
        q5 = self.qkv_local.view(B, self.S_loc, 3, self.H, self.Dh)
        q = q5[:, :, 0]
        out = lse = None
        if self.mode == "peer":
            from .peer_memory import pull_rows
            P, r, Si, St = self.P, self.rank, self.Si_loc, self.St_loc
            dev, dt = self.qkv_local.device, self.qkv_local.dtype
            es = self.qkv_local.element_size()
            o4 = self.attn.view(B, self.S_loc, self.H, self.Dh)
            self.arena.barrier()                                  # every rank's K/V shard is in place
            if P == 1:
                attention(q, q5[:, :, 1], q5[:, :, 2], kv_lens=self._shard_kv_lens(kv_lens, r), out=o4)
            else:
                main = torch.cuda.current_stream(dev)
                overlap = two_launches_pay(B, self.S_loc, self.H)
                if self._side is None or self._overlap != overlap:
                    self._side, self._overlap = torch.cuda.Stream(dev), overlap
                    # rows in the gathered buffer: image rows in rank order, then text rows in rank order, so that
                    # valid keys (text is padded at the end of the global text) stay a prefix.  The overlapped
                    # form leaves the own shard out (it is read in place by the first launch).
                    self._srcs = [s for s in range(P) if s != r] if overlap else list(range(P))
                    n = len(self._srcs)
                    self._gath = torch.empty(B, n * self.S_loc, 2 * HD, dtype=dt, device=dev)
                    self._srcs_t = torch.tensor(self._srcs, device=dev, dtype=torch.int32)
                n = len(self._srcs)
                pitch = 3 * HD * es

                def pull(j, src):
                    for b in range(B):
                        base = self.qkv.ptrs[src] + ((b * self.S_loc) * 3 * HD + HD) * es
                        pull_rows(self._gath[b, j * Si:(j + 1) * Si], base, pitch)
                        if St:
                            t0 = n * Si + j * St
                            pull_rows(self._gath[b, t0:t0 + St], base + Si * pitch, pitch)
                self._side.wait_stream(main)
                with torch.cuda.stream(self._side):
                    for j, src in enumerate(self._srcs):
                        if src != r:
                            pull(j, src)
                g5 = self._gath.view(B, n * self.S_loc, 2, self.H, self.Dh)
                if overlap:
                    # big grids: the own shard is attended to in place while the pulls run; the second launch
                    # takes the remote rows and combines both results in its epilogue
                    _, lse0 = attention(q, q5[:, :, 1], q5[:, :, 2], kv_lens=self._shard_kv_lens(kv_lens, r), return_lse=True, out=o4)
                    main.wait_stream(self._side)
                    rem_lens = None
                    if kv_lens is not None:
                        txt = (kv_lens[:, None] - self.S_img - self._srcs_t[None] * St).clamp(0, St).sum(dim=1)
                        rem_lens = (n * Si + txt).to(torch.int32)
                    attention(q, g5[:, :, 0], g5[:, :, 1], kv_lens=rem_lens, merge_prev=(o4, lse0), out=o4)
                else:
                    # small grids (a launch is a wave or two): ONE launch over all keys in global order; the own
                    # shard is copied locally on the main stream while the side stream pulls the others
                    pull(r, r)
                    main.wait_stream(self._side)
                    attention(q, g5[:, :, 0], g5[:, :, 1], kv_lens=kv_lens.to(torch.int32) if kv_lens is not None else None, out=o4)
            self.arena.barrier()                                  # shards may be overwritten by the next layer
            return self.attn[:, :self.Si_loc], self.attn[:, self.Si_loc:]
        else:
            comm = RingComm(self.group.device_group)
            k, v = q5[:, :, 1].contiguous(), q5[:, :, 2].contiguous()
            for step in range(self.P):
                src = (self.rank - step) % self.P
                if step + 1 < self.P:
                    nk, nv_ = comm.send_recv(k), comm.send_recv(v)
                    comm.commit()
                o_b, lse_b = attention(q, k, v, kv_lens=self._shard_kv_lens(kv_lens, src), return_lse=True)
                out, lse = merge_attention(out, lse, o_b, lse_b)
                if step + 1 < self.P:
                    comm.wait()
                    k, v = nk, nv_
        self.attn.copy_(out.reshape(B, self.S_loc, HD))
        return self.attn[:, :self.Si_loc], self.attn[:, self.Si_loc:]

    def close(self):
        if self.arena is not None:
            self.arena.close()
            self.arena = None
