"""Wan2.x-style video DiT on the fused sm_100a ops.

Structure of ``WanTransformer3DModel`` (vllm_omni/diffusion/models/wan2_2/wan2_2_transformer.py:
728-990): (1,2,2) patch embedding, text MLP, timestep MLP whose 6*D projection is added to a
learned ``scale_shift_table`` per block, 40 blocks of [modulated LayerNorm -> self attention
with RMSNorm over the full q/k width and 3-D RoPE -> gated residual; LayerNorm -> cross attention
to the text tokens -> residual; modulated LayerNorm -> GELU FFN -> gated residual], modulated
output norm and projection.  Sequence parallelism shards the video tokens; cross attention stays
local because the text is replicated.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ....ops import fused
from ....ops.attention import attention
from ...layers.linear import FusedLinear
from ..qwen_image.transformer import timestep_sinusoid


@dataclass
class WanTransformerConfig:
    patch_size: tuple = (1, 2, 2)
    num_attention_heads: int = 40
    attention_head_dim: int = 128
    in_channels: int = 16
    out_channels: int = 16
    text_dim: int = 4096
    freq_dim: int = 256
    ffn_dim: int = 13824
    num_layers: int = 40
    eps: float = 1e-6
    rope_max_seq_len: int = 1024

    @property
    def inner_dim(self):
        return self.num_attention_heads * self.attention_head_dim

    @classmethod
    def from_dict(cls, d):
        keys = set(cls.__dataclass_fields__)
        return cls(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in d.items() if k in keys})


def wan_rope_angles(f: int, h: int, w: int, head_dim: int, theta: float = 10000.0) -> torch.Tensor:
    """[f*h*w, head_dim/2] angles: the frequency range is split (d - 2*(d//3), d//3, d//3) over
    (frame, height, width)."""
    d = head_dim
    dh = dw = 2 * (d // 6)
    dt = d - dh - dw

    def ang(n, dim):
        inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
        return torch.outer(torch.arange(n, dtype=torch.float32), inv)
    a = torch.cat([ang(f, dt)[:, None, None, :].expand(f, h, w, -1), ang(h, dh)[None, :, None, :].expand(f, h, w, -1),
                   ang(w, dw)[None, None, :, :].expand(f, h, w, -1)], dim=-1)
    return a.reshape(f * h * w, d // 2)


class WanBlock(nn.Module):
    def __init__(self, cfg: WanTransformerConfig, dtype, device):
        super().__init__()
        D = cfg.inner_dim
        P = lambda *s: nn.Parameter(torch.ones(*s, dtype=dtype, device=device), requires_grad=False)
        self.scale_shift_table = nn.Parameter(torch.randn(6, D, dtype=dtype, device=device) / D ** 0.5,
                                              requires_grad=False)
        self.attn1_qkv = FusedLinear(D, 3 * D, dtype=dtype, device=device)
        self.attn1_norm_q, self.attn1_norm_k = P(D), P(D)
        self.attn1_out = FusedLinear(D, D, dtype=dtype, device=device)
        self.norm2_w = P(D)
        self.norm2_b = nn.Parameter(torch.zeros(D, dtype=dtype, device=device), requires_grad=False)
        self.attn2_q = FusedLinear(D, D, dtype=dtype, device=device)
        self.attn2_kv = FusedLinear(D, 2 * D, dtype=dtype, device=device)
        self.attn2_norm_q, self.attn2_norm_k = P(D), P(D)
        self.attn2_out = FusedLinear(D, D, dtype=dtype, device=device)
        self.ffn_up = FusedLinear(D, cfg.ffn_dim, dtype=dtype, device=device)
        self.ffn_down = FusedLinear(cfg.ffn_dim, D, dtype=dtype, device=device)


class WanTransformer3DModel(nn.Module):
    graph_safe_forward = True          # stateless between calls of one signature: may be replayed from a CUDA graph
    def __init__(self, cfg: WanTransformerConfig | None = None, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg = cfg or WanTransformerConfig()
        self.dtype_ = dtype
        D = cfg.inner_dim
        pt, ph, pw = cfg.patch_size
        self.patch_embedding = FusedLinear(cfg.in_channels * pt * ph * pw, D, dtype=dtype, device=device)
        self.text_1 = FusedLinear(cfg.text_dim, D, dtype=dtype, device=device)
        self.text_2 = FusedLinear(D, D, dtype=dtype, device=device)
        self.time_1 = FusedLinear(cfg.freq_dim, D, dtype=dtype, device=device)
        self.time_2 = FusedLinear(D, D, dtype=dtype, device=device)
        self.time_proj = FusedLinear(D, 6 * D, dtype=dtype, device=device)
        self.blocks = nn.ModuleList([WanBlock(cfg, dtype, device) for _ in range(cfg.num_layers)])
        self.out_table = nn.Parameter(torch.randn(2, D, dtype=dtype, device=device) / D ** 0.5, requires_grad=False)
        self.proj_out = FusedLinear(D, cfg.out_channels * pt * ph * pw, dtype=dtype, device=device)
        self.tp_group = self.tp_reduce = None      # tensor parallelism: heads and FFN columns split over the group
        self.sp = None                   # SequenceParallelAttention when the sequence is sharded
        self.sp_style = "attention"
        self._sp_valid_len = None
        self.stack_hook = None            # cache backends: called once per step with a BlockStack over the blocks
        self._rope = {}

    # -------------------------------------------------------------- tensor parallelism
    def enable_tensor_parallel(self, group, mode: str | None = None) -> None:
        """Heads of both attentions and the FFN columns are split over ``group``; the three output
        projections become row-parallel (partial sums finished by ``RowParallelReduce``, with the
        AdaLN gate and the residual applied once by the reduce).  The q / k RMSNorms of Wan run over ALL
        heads' channels, so each rank norms its slice with the mean square summed over the group: one
        small all-reduce of per-row sums for q and k together (the reference's ``DistributedRMSNorm``,
        vllm_omni/diffusion/models/wan2_2/wan2_2_transformer.py)."""
        from ....parallel.tensor_parallel import RowParallelReduce
        n, r = group.world_size, group.rank_in_group
        if n == 1:
            return
        cfg = self.cfg
        D, H = cfg.inner_dim, cfg.num_attention_heads
        if H % n or cfg.ffn_dim % n:
            raise ValueError(f"heads ({H}) and ffn_dim ({cfg.ffn_dim}) must be divisible by tensor_parallel_size ({n})")
        Dl, Fl = D // n, cfg.ffn_dim // n

        def cols(lin, parts):           # keep this rank's slice of each of the `parts` equal row groups of the weight
            w, b = lin.weight.data, (lin.bias.data if lin.bias is not None else None)
            per = w.shape[0] // parts
            sl = per // n
            idx = torch.cat([torch.arange(g * per + r * sl, g * per + (r + 1) * sl) for g in range(parts)]).to(w.device)
            new = FusedLinear(w.shape[1], idx.numel(), bias=b is not None, dtype=w.dtype, device=w.device)
            new.weight.data.copy_(w[idx])
            if b is not None:
                new.bias.data.copy_(b[idx])
            return new

        def rows(lin, width):           # keep this rank's input features; the bias is added once, by the reduce
            w = lin.weight.data
            new = FusedLinear(width, w.shape[0], bias=False, dtype=w.dtype, device=w.device)
            new.weight.data.copy_(w[:, r * width:(r + 1) * width])
            new.full_bias = lin.bias.data.clone() if lin.bias is not None else None
            return new
        sl = slice(r * Dl, (r + 1) * Dl)
        for blk in self.blocks:
            blk.attn1_qkv, blk.attn1_out = cols(blk.attn1_qkv, 3), rows(blk.attn1_out, Dl)
            blk.attn2_q, blk.attn2_kv, blk.attn2_out = cols(blk.attn2_q, 1), cols(blk.attn2_kv, 2), rows(blk.attn2_out, Dl)
            blk.ffn_up, blk.ffn_down = cols(blk.ffn_up, 1), rows(blk.ffn_down, Fl)
            for nm in ("attn1_norm_q", "attn1_norm_k", "attn2_norm_q", "attn2_norm_k"):
                setattr(blk, nm, nn.Parameter(getattr(blk, nm).data[sl].clone(), requires_grad=False))
        self.tp_group, self.tp_reduce = group, RowParallelReduce(group, mode)

    def _rms_across_ranks(self, parts, weights):
        """RMSNorm of tensors whose channel dimension is split over the TP group: ``parts`` are this rank's
        [.., D/P] slices; their mean squares are summed over the group in one all-reduce."""
        D, eps = self.cfg.inner_dim, self.cfg.eps
        ss = [p.float().pow(2).sum(-1, keepdim=True) for p in parts]
        flat = torch.cat([t.reshape(-1) for t in ss])
        self.tp_group.all_reduce(flat)
        out, o = [], 0
        for p, t, w in zip(parts, ss, weights):
            tot = flat[o:o + t.numel()].view_as(t)
            o += t.numel()
            out.append((p.float() * torch.rsqrt(tot / D + eps) * w.float()).to(p.dtype))
        return out

    def _row_out(self, lin, a, x, gate=None):
        """x += gate * (lin(a) summed over the TP group + bias)."""
        if self.tp_reduce is None:
            lin(a, residual=x, gate=gate, out=x)
        else:
            self.tp_reduce.linear(lin, a, bias=getattr(lin, "full_bias", None), gate=gate, residual=x, out=x)

    # -------------------------------------------------------------- patchify
    def patchify(self, x):          # [B, C, T, H, W] -> [B, S, C*pt*ph*pw], grid
        pt, ph, pw = self.cfg.patch_size
        B, C, T, H, W = x.shape
        g = (T // pt, H // ph, W // pw)
        x = x.view(B, C, g[0], pt, g[1], ph, g[2], pw).permute(0, 2, 4, 6, 1, 3, 5, 7)
        return x.reshape(B, g[0] * g[1] * g[2], C * pt * ph * pw), g

    def unpatchify(self, y, g):     # inverse
        pt, ph, pw = self.cfg.patch_size
        B = y.shape[0]
        C = self.cfg.out_channels
        y = y.view(B, g[0], g[1], g[2], C, pt, ph, pw).permute(0, 4, 1, 5, 2, 6, 3, 7)
        return y.reshape(B, C, g[0] * pt, g[1] * ph, g[2] * pw)

    def rope(self, g, device):
        key = (g, str(device))
        if key not in self._rope:
            a = wan_rope_angles(*g, self.cfg.attention_head_dim)
            self._rope[key] = (a.cos().contiguous().to(device), a.sin().contiguous().to(device))
        return self._rope[key]

    # -------------------------------------------------------------- forward
    def block_forward(self, blk: WanBlock, x, ctx, e6, cos, sin):
        """x [B,S,D] in place; ctx [B,L,D] text; e6 [B,6,D] = temb projection."""
        cfg = self.cfg
        D, H, Dh = cfg.inner_dim, cfg.num_attention_heads, cfg.attention_head_dim
        B, S, _ = x.shape
        mod = (blk.scale_shift_table[None].float() + e6.float()).to(x.dtype).reshape(B, 6 * D)
        xn = fused.norm_modulate(x, shift=mod[:, 0:D], scale=mod[:, D:2 * D], eps=cfg.eps)
        tp = self.tp_group is not None
        if tp:
            H = H // self.tp_group.world_size
        Dl = H * Dh                                                           # this rank's attention width
        qkv = blk.attn1_qkv(xn)                                              # [B,S,3*Dl]
        if tp:
            q, k = self._rms_across_ranks([qkv[..., :Dl], qkv[..., Dl:2 * Dl]], [blk.attn1_norm_q, blk.attn1_norm_k])
        else:
            q = fused.norm_modulate(qkv[..., :D].contiguous(), weight=blk.attn1_norm_q, rms=True, eps=cfg.eps)
            k = fused.norm_modulate(qkv[..., D:2 * D].contiguous(), weight=blk.attn1_norm_k, rms=True, eps=cfg.eps)
        qk = torch.cat([q, k, qkv[..., 2 * Dl:]], dim=-1).contiguous()
        fused.qk_norm_rope_(qk, H, H, Dh, cos=cos, sin=sin, interleaved=True, eps=cfg.eps)
        q5 = qk.view(B, S, 3, H, Dh)
        if self.sp is not None:
            # sequence parallel: x holds this rank's rows; only self-attention sees the other ranks
            o = self.sp(q5, valid_len=self._sp_valid_len).reshape(B, S, Dl)
        else:
            o = attention(q5[:, :, 0], q5[:, :, 1], q5[:, :, 2]).reshape(B, S, Dl)
        self._row_out(blk.attn1_out, o, x, gate=mod[:, 2 * D:3 * D])
        xn = fused.norm_modulate(x, weight=blk.norm2_w, bias=blk.norm2_b, eps=cfg.eps)
        kv = blk.attn2_kv(ctx)
        L = ctx.shape[1]
        if tp:
            q, = self._rms_across_ranks([blk.attn2_q(xn)], [blk.attn2_norm_q])
            k2, = self._rms_across_ranks([kv[..., :Dl]], [blk.attn2_norm_k])
        else:
            q = fused.norm_modulate(blk.attn2_q(xn), weight=blk.attn2_norm_q, rms=True, eps=cfg.eps)
            k2 = fused.norm_modulate(kv[..., :D].contiguous(), weight=blk.attn2_norm_k, rms=True, eps=cfg.eps)
        o = attention(q.reshape(B, S, H, Dh), k2.reshape(B, L, H, Dh), kv[..., Dl:].reshape(B, L, H, Dh)).reshape(B, S, Dl)
        self._row_out(blk.attn2_out, o, x)
        xn = fused.norm_modulate(x, shift=mod[:, 3 * D:4 * D], scale=mod[:, 4 * D:5 * D], eps=cfg.eps)
        self._row_out(blk.ffn_down, blk.ffn_up(xn, act="gelu_tanh"), x, gate=mod[:, 5 * D:6 * D])
        return x

    def forward(self, hidden_states, timestep, encoder_hidden_states, **_):
        """hidden_states [B, C, T, H, W]; timestep [B] (0..1000); encoder_hidden_states [B, L, text_dim]."""
        cfg, D = self.cfg, self.cfg.inner_dim
        tokens, g = self.patchify(hidden_states.to(self.dtype_))
        B = tokens.shape[0]
        x = self.patch_embedding(tokens.contiguous())
        cos, sin = self.rope(g, x.device)
        S_full = x.shape[1]
        if self.sp is not None:
            # keep S / P rows (zero rows pad S up to a multiple of P and are masked as keys)
            x, _ = self.sp.shard_rows(x, dim=1)
            rows = self.sp.local_rows(S_full)
            pad = x.shape[1] - cos[rows].shape[0]
            cos = torch.cat([cos[rows], cos.new_ones(pad, cos.shape[1])]) if pad else cos[rows].contiguous()
            sin = torch.cat([sin[rows], sin.new_zeros(pad, sin.shape[1])]) if pad else sin[rows].contiguous()
            self._sp_valid_len = S_full if S_full % self.sp.P else None
        ctx = self.text_2(self.text_1(encoder_hidden_states.to(self.dtype_), act="gelu_tanh"))
        temb = self.time_2(self.time_1(timestep_sinusoid(timestep, cfg.freq_dim, scale=1.0).to(self.dtype_), act="silu"))
        e6 = self.time_proj(F.silu(temb)).view(B, 6, D)
        def run(states, a, b):
            for blk in self.blocks[a:b]:
                self.block_forward(blk, states[0], ctx, e6, cos, sin)        # in place
            return states
        if self.stack_hook is not None:
            from ...cache.base import BlockStack
            probe = fused.norm_modulate(x, shift=e6[:, 0].contiguous(), scale=e6[:, 1].contiguous(), eps=cfg.eps)
            (x,) = self.stack_hook(BlockStack(len(self.blocks), (x,), probe, run))
        else:
            run((x,), 0, len(self.blocks))
        om = (self.out_table[None].float() + temb[:, None].float()).to(x.dtype)      # [B,2,D]: shift, scale
        xn = fused.norm_modulate(x, shift=om[:, 0].contiguous(), scale=om[:, 1].contiguous(), eps=cfg.eps)
        y = self.proj_out(xn)
        if self.sp is not None:
            y = self.sp.gather_rows(y, S_full, dim=1)
        return self.unpatchify(y.contiguous(), g)

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        """diffusers ``WanTransformer3DModel`` names; q/k/v and k/v are stacked into the fused
        projections."""
        cfg, D = self.cfg, self.cfg.inner_dim
        params = dict(self.named_parameters())
        simple = {"condition_embedder.text_embedder.linear_1": "text_1", "condition_embedder.text_embedder.linear_2": "text_2",
                  "condition_embedder.time_embedder.linear_1": "time_1", "condition_embedder.time_embedder.linear_2": "time_2",
                  "condition_embedder.time_proj": "time_proj", "proj_out": "proj_out"}
        loaded = set()
        for name, w in weights:
            tgt, sl = None, None
            base, _, leaf = name.rpartition(".")
            if base in simple:
                tgt = f"{simple[base]}.{leaf}"
                if base == "proj_out":
                    # the checkpoint emits a patch as (pt, ph, pw, c); ``unpatchify`` reads (c, pt, ph, pw)
                    C = cfg.out_channels
                    w = w.reshape(w.shape[0] // C, C, *w.shape[1:]).transpose(0, 1).reshape(w.shape)
            elif name == "patch_embedding.weight":
                tgt, w = "patch_embedding.weight", w.reshape(w.shape[0], -1)
            elif name == "patch_embedding.bias":
                tgt = "patch_embedding.bias"
            elif name == "scale_shift_table":
                tgt, w = "out_table", w.reshape(2, D)
            elif name.startswith("blocks."):
                p = name.split(".")
                i, rest = int(p[1]), ".".join(p[2:])
                pre = f"blocks.{i}."
                qkv = {"attn1.to_q": 0, "attn1.to_k": 1, "attn1.to_v": 2}
                kv = {"attn2.to_k": 0, "attn2.to_v": 1}
                b2, _, lf = rest.rpartition(".")
                if b2 in qkv:
                    tgt, sl = pre + f"attn1_qkv.{lf}", (qkv[b2] * D, (qkv[b2] + 1) * D)
                elif b2 in kv:
                    tgt, sl = pre + f"attn2_kv.{lf}", (kv[b2] * D, (kv[b2] + 1) * D)
                else:
                    m = {"attn1.to_out.0": "attn1_out", "attn2.to_q": "attn2_q", "attn2.to_out.0": "attn2_out",
                         "ffn.net.0.proj": "ffn_up", "ffn.net.2": "ffn_down"}
                    if b2 in m:
                        tgt = pre + f"{m[b2]}.{lf}"
                    elif rest == "scale_shift_table":
                        tgt, w = pre + "scale_shift_table", w.reshape(6, D)
                    elif rest in ("attn1.norm_q.weight", "attn1.norm_k.weight", "attn2.norm_q.weight", "attn2.norm_k.weight"):
                        tgt = pre + rest.replace(".norm_", "_norm_").replace(".weight", "")
                    elif rest == "norm2.weight":
                        tgt = pre + "norm2_w"
                    elif rest == "norm2.bias":
                        tgt = pre + "norm2_b"
            if tgt is None or tgt not in params:
                continue
            dst = params[tgt] if sl is None else params[tgt][sl[0]:sl[1]]
            dst.copy_(w.to(dst.dtype).reshape(dst.shape))
            loaded.add(name)
        return loaded
