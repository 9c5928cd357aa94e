"""Ulysses sequence parallelism for joint (image + text) attention.

Each rank owns S_img/P image rows and S_txt/P text rows of every sample (text is sharded
like the image; the reference keeps it replicated and head-sliced,
vllm_omni/diffusion/attention/parallel/ulysses.py:61-238, which costs P-fold redundant text
compute).  Attention needs every row but only H/P heads per rank, i.e. a head<->sequence
all-to-all before and after.

``mode="fused"`` (GPU): no collective calls and no layout copies.
  * the QKV GEMM epilogue stores each head group straight into its owner rank's joint
    ``[B, S_img+S_txt, 3, H/P, Dh]`` buffer over NVLink (csrc/gemm_sm100.cu scatter epilogue);
  * the attention epilogue stores each output row straight into the owner rank's
    ``[B, S_loc, H, Dh]`` buffer at this rank's head offset (csrc/attention_sm100.cu);
  * no barrier kernels: every producer launch reports one arrival to each rank once its peer
    stores are out, and the consumer kernel (q/k norm + rope after the QKV exchange, the
    out-projection GEMM after the attention exchange) waits for this use's arrivals itself, with a
    bounded spin (csrc/peer_signal.cuh).  Projections that cannot carry the signal (fp8, LoRA)
    fall back to the bounded-wait barrier kernel of csrc/peer_rt.cu.
``mode="nccl"``: the same data movement with ``all_to_all_single`` + permutes — the baseline
the fused path is measured against, and the path CPU (Gloo) tests run.
"""
from __future__ import annotations

import os

import torch

from ..ops import fused
from ..ops.attention import attention
from .comm import all_to_all_4d, all_to_all_5d


class UlyssesJointAttention:
    def __init__(self, group, num_heads: int, head_dim: int, mode: str | None = None):
        self.group = group
        self.P, self.rank = group.world_size, group.rank_in_group
        if num_heads % self.P:
            raise ValueError(f"num_heads ({num_heads}) must be divisible by the Ulysses degree ({self.P})")
        self.H, self.Dh, self.Hp = num_heads, head_dim, num_heads // self.P
        self.mode = mode or ("fused" if torch.cuda.is_available() else "nccl")
        # one launch for the image and text QKV projections (OMNI_SP_PAIR_QKV=0 keeps them apart)
        self.pair_streams = os.environ.get("OMNI_SP_PAIR_QKV", "1") == "1"
        # arrivals consumed inside the next kernel (OMNI_SP_FLAGS=0: barrier kernels instead)
        self.use_flags = os.environ.get("OMNI_SP_FLAGS", "1") == "1"
        self._out_wait = None
        self.arena = None
        self._key = None

    # ------------------------------------------------------------------ buffers
    def setup(self, B: int, Si_loc: int, St_loc: int, device, dtype):
        key = (B, Si_loc, St_loc, str(device), dtype)
        if self._key == key:
            return
        self._key = key
        self.B, self.Si_loc, self.St_loc = B, Si_loc, St_loc
        self.S_img, self.S_txt = Si_loc * self.P, St_loc * self.P
        self.S_tot = self.S_img + self.S_txt
        G = self.Hp * self.Dh
        if self.mode == "fused":
            from .peer_memory import PeerArena, SignalChannel
            if self.arena is not None:
                self.arena.close()
            es = torch.empty(0, dtype=dtype).element_size()
            need = (B * self.S_tot * 3 * G + B * (Si_loc + St_loc) * self.H * self.Dh) * es + 16384
            self.arena = PeerArena(self.group, need, device)
            self.ch_qkv = SignalChannel(self.arena)      # QKV rows arrived -> q/k norm + rope
            self.ch_attn = SignalChannel(self.arena)     # attention rows arrived -> out-projection
            self.group.barrier()                         # counters are zeroed everywhere before first use
            self.joint = self.arena.alloc((B, self.S_tot, 3 * G), dtype)
            self.attn_img = self.arena.alloc((B, Si_loc, self.H * self.Dh), dtype)
            self.attn_txt = self.arena.alloc((B, St_loc, self.H * self.Dh), dtype)
            ld = 3 * G
            self._img_scatter = (self.P, G, self.joint.peer_ptrs(self.rank * Si_loc * ld * es), ld)
            self._txt_scatter = (self.P, G, self.joint.peer_ptrs((self.S_img + self.rank * St_loc) * ld * es), ld)
            hoff = self.rank * G * es
            HD = self.H * self.Dh
            self._attn_scatter = dict(n_peers=self.P, rows_per_rank=Si_loc, rows_per_rank2=max(St_loc, 1),
                                      split=self.S_img, o_ptrs=self.attn_img.peer_ptrs(hoff),
                                      o2_ptrs=self.attn_txt.peer_ptrs(hoff), o_strides=(HD, self.Dh, Si_loc * HD),
                                      o2_strides=(HD, self.Dh, St_loc * HD))
            self.joint_local = self.joint.local
        else:
            e = lambda *s: torch.empty(*s, dtype=dtype, device=device)
            self.joint_local = e(B, self.S_tot, 3 * G)
            self.qkv_img = e(B, Si_loc, 3 * self.H * self.Dh)
            self.qkv_txt = e(B, St_loc, 3 * self.H * self.Dh)

    # ------------------------------------------------------------------ per block
    def project_qkv(self, img_lin, xn_img, txt_lin, xn_txt):
        """QKV projections of the local rows; afterwards ``joint_local`` holds q,k,v of ALL rows
        for this rank's heads."""
        G, B = self.Hp * self.Dh, self.B
        if self.mode == "fused":
            bs = self.S_tot * 3 * G
            plain = all(l.fp8 is None and not l.lora for l in (img_lin, txt_lin))
            # the block's other linears must be able to carry the wait as well (set by the model)
            self._flags_now = flags = self.use_flags and plain and getattr(self, "block_plain", True)
            sig = self.ch_qkv.signal() if flags else None
            if self.St_loc and plain and self.pair_streams:
                # image and text projection in one launch; each carries its own scatter pointers
                from ..ops import gemm
                gemm.linear_pair(
                    dict(x=xn_img, w=img_lin.weight, bias=img_lin.bias, scatter=self._img_scatter,
                         out_rows_per_batch=self.Si_loc, out_batch_stride=bs),
                    dict(x=xn_txt, w=txt_lin.weight, bias=txt_lin.bias, scatter=self._txt_scatter,
                         out_rows_per_batch=self.St_loc, out_batch_stride=bs), sync=sig)
            elif flags:
                # the last launch reports for both: the first one's stores are complete at its end
                img_lin(xn_img, scatter=self._img_scatter, out_rows_per_batch=self.Si_loc, out_batch_stride=bs,
                        sync=None if self.St_loc else sig)
                if self.St_loc:
                    txt_lin(xn_txt, scatter=self._txt_scatter, out_rows_per_batch=self.St_loc, out_batch_stride=bs,
                            sync=sig)
            else:
                img_lin(xn_img, scatter=self._img_scatter, out_rows_per_batch=self.Si_loc, out_batch_stride=bs)
                if self.St_loc:
                    txt_lin(xn_txt, scatter=self._txt_scatter, out_rows_per_batch=self.St_loc, out_batch_stride=bs)
            if not flags:
                self.arena.barrier()
            return
        grp = self.group.device_group
        img_lin(xn_img, out=self.qkv_img)
        q = all_to_all_5d(self.qkv_img.view(B, self.Si_loc, 3, self.H, self.Dh), 3, 1, grp)
        self.joint_local[:, :self.S_img].copy_(q.reshape(B, self.S_img, 3 * G))
        if self.St_loc:
            txt_lin(xn_txt, out=self.qkv_txt)
            t = all_to_all_5d(self.qkv_txt.view(B, self.St_loc, 3, self.H, self.Dh), 3, 1, grp)
            self.joint_local[:, self.S_img:].copy_(t.reshape(B, self.S_txt, 3 * G))

    def norm_rope(self, wq, wk, wq_txt, wk_txt, cos, sin, eps):
        wait = self.ch_qkv.wait() if self.mode == "fused" and getattr(self, "_flags_now", False) else None
        fused.qk_norm_rope_(self.joint_local, self.Hp, self.Hp, self.Dh, wq=wq, wk=wk, wq_alt=wq_txt, wk_alt=wk_txt,
                            s_alt=self.S_img, cos=cos, sin=sin, interleaved=True, eps=eps, sync=wait)

    def attend(self, kv_lens, ws):
        """Joint attention over this rank's heads; returns (attn_img [B,Si_loc,H*Dh],
        attn_txt [B,St_loc,H*Dh]) holding ALL heads of the local rows."""
        B = self.B
        q5 = self.joint_local.view(B, self.S_tot, 3, self.Hp, self.Dh)
        if self.mode == "fused":
            if getattr(self, "_flags_now", False):
                attention(q5[:, :, 0], q5[:, :, 1], q5[:, :, 2], kv_lens=kv_lens, scatter=self._attn_scatter,
                          sync=self.ch_attn.signal())
                self._out_wait = self.ch_attn.wait()      # the out-projection GEMM waits for the rows itself
            else:
                attention(q5[:, :, 0], q5[:, :, 1], q5[:, :, 2], kv_lens=kv_lens, scatter=self._attn_scatter)
                self.arena.barrier()
            return self.attn_img.local, self.attn_txt.local
        o = attention(q5[:, :, 0], q5[:, :, 1], q5[:, :, 2], kv_lens=kv_lens)     # [B, S_tot, Hp, Dh]
        grp = self.group.device_group
        oi = all_to_all_4d(o[:, :self.S_img].contiguous(), 1, 2, grp).reshape(B, self.Si_loc, self.H * self.Dh)
        ot = None
        if self.St_loc:
            ot = all_to_all_4d(o[:, self.S_img:].contiguous(), 1, 2, grp).reshape(B, self.St_loc, self.H * self.Dh)
        return oi, ot

    def take_out_wait(self):
        """The arrivals the first GEMM that reads the attention output has to wait for (``OmniSync``),
        or None when a barrier kernel already ordered the exchange.  Handed out once per block."""
        w, self._out_wait = self._out_wait, None
        return w

    def close(self):
        if self.arena is not None:
            self.arena.close()
            self.arena = None
