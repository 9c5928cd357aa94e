"""Single-stream generation transformer of the Bagel DiT stage
(vllm_omni/diffusion/models/bagel/bagel_transformer.py): one sequence [image tokens | text tokens],
per layer timestep-conditioned scale/gate, RMSNorm, attention with q/k RMSNorm and 3-axis RoPE,
SwiGLU MLP with merged ``w13``.  Every attention layer can attend to a key/value prefix handed
over by the upstream AR stage (``past_key_values``), which is how the reference's ``NaiveCache``
injects the prompt context.  Declares a sequence-parallel plan."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ....ops import fused
from ....ops.attention import attention
from ....parallel.sp_plan import SequenceParallelInput, SequenceParallelOutput
from ...layers.linear import FusedLinear
from ..flux.transformer import flux_rope_angles
from ..qwen_image.transformer import TimestepEmbedder


@dataclass
class BagelTransformerConfig:
    dim: int = 3840
    n_layers: int = 30
    n_heads: int = 30
    head_dim: int = 128
    ffn_dim: int = 10240
    in_channels: int = 64
    out_channels: int = 16
    cap_feat_dim: int = 2560
    axes_dims_rope: tuple = (32, 48, 48)
    rope_theta: float = 256.0
    eps: float = 1e-5
    past_kv_layers: bool = False

    @classmethod
    def from_dict(cls, d):
        keys = set(cls.__dataclass_fields__)
        return cls(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in d.items() if k in keys})


class BagelBlock(nn.Module):
    def __init__(self, c: BagelTransformerConfig, dtype, device):
        super().__init__()
        D, H, Dh = c.dim, c.n_heads, c.head_dim
        P = lambda *s: nn.Parameter(torch.ones(*s, dtype=dtype, device=device), requires_grad=False)
        self.adaln = FusedLinear(min(D, 256), 4 * D, dtype=dtype, device=device)
        self.attn_norm1, self.attn_norm2, self.ffn_norm1, self.ffn_norm2 = P(D), P(D), P(D), P(D)
        self.qkv = FusedLinear(D, 3 * H * Dh, bias=False, dtype=dtype, device=device)
        self.q_norm, self.k_norm = P(Dh), P(Dh)
        self.out = FusedLinear(H * Dh, D, bias=False, dtype=dtype, device=device)
        self.w13 = FusedLinear(D, 2 * c.ffn_dim, bias=False, dtype=dtype, device=device)
        self.w2 = FusedLinear(c.ffn_dim, D, bias=False, dtype=dtype, device=device)


class BagelTransformer2DModel(nn.Module):
    _sp_plan = {"": {"hidden_states": SequenceParallelInput(split_dim=1, expected_dims=3, auto_pad=True)},
                "proj_out": SequenceParallelOutput(gather_dim=1)}

    def __init__(self, cfg: BagelTransformerConfig | None = None, dtype=torch.bfloat16, device=None, tp_size: int = 1):
        super().__init__()
        self.cfg = c = cfg or BagelTransformerConfig()
        self.validate_tp(c, tp_size)
        self.dtype_ = dtype
        D = c.dim
        self.x_embedder = FusedLinear(c.in_channels, D, dtype=dtype, device=device)
        self.cap_norm = nn.Parameter(torch.ones(c.cap_feat_dim, dtype=dtype, device=device), requires_grad=False)
        self.cap_embedder = FusedLinear(c.cap_feat_dim, D, dtype=dtype, device=device)
        self.t_embedder = TimestepEmbedder(min(D, 256), dtype, device)
        self.layers = nn.ModuleList([BagelBlock(c, dtype, device) for _ in range(c.n_layers)])
        self.final_adaln = FusedLinear(min(D, 256), D, dtype=dtype, device=device)
        self.proj_out = FusedLinear(D, c.out_channels * 4, dtype=dtype, device=device)
        self.block_hook = None
        self.sp = None                   # SequenceParallelAttention when the joint sequence is sharded
        self.sp_style = "attention"
        self._ang = {}

    @staticmethod
    def validate_tp(c, tp):
        if tp > 1 and (c.n_heads % tp or c.ffn_dim % tp):
            raise ValueError(f"n_heads ({c.n_heads}) and ffn_dim ({c.ffn_dim}) must be divisible by TP size {tp}")

    def forward(self, hidden_states, encoder_hidden_states, timestep, img_shapes, txt_seq_lens=None,
                past_key_values=None, **_):
        c = self.cfg
        D, H, Dh = c.dim, c.n_heads, c.head_dim
        B, S_img, S_txt = hidden_states.shape[0], hidden_states.shape[1], encoder_hidden_states.shape[1]
        dev = hidden_states.device
        _, h, w = img_shapes
        key = (h, w, S_txt, str(dev))
        if key not in self._ang:
            a = flux_rope_angles(h, w, S_txt, c.axes_dims_rope, c.rope_theta)
            self._ang[key] = (a.cos().contiguous().to(dev), a.sin().contiguous().to(dev))
        cos, sin = self._ang[key]
        kv_lens = None
        if txt_seq_lens is not None and any(int(l) != S_txt for l in txt_seq_lens) and past_key_values is None:
            kv_lens = torch.tensor([S_img + int(l) for l in txt_seq_lens], dtype=torch.int32, device=dev)
        x = self.x_embedder(hidden_states.to(self.dtype_))
        cap = self.cap_embedder(fused.norm_modulate(encoder_hidden_states.to(self.dtype_).contiguous(),
                                                    weight=self.cap_norm, rms=True, eps=c.eps))
        x = torch.cat([x, cap], dim=1).contiguous()
        S_full = x.shape[1]
        sp = self.sp if past_key_values is None else None
        sp_lens = None
        if sp is not None:
            # rows of the joint [image, text] sequence are split over the SP group; text padding and
            # the zero rows that round S up to a multiple of P are masked as keys
            x, _ = sp.shard_rows(x, dim=1)
            rows = sp.local_rows(S_full)
            pad = x.shape[1] - cos[rows].shape[0]
            cos = torch.cat([cos[rows], cos.new_ones(pad, cos.shape[1])]) if pad else cos[rows].contiguous()
            sin = torch.cat([sin[rows], sin.new_zeros(pad, sin.shape[1])]) if pad else sin[rows].contiguous()
            if kv_lens is not None:
                sp_lens = kv_lens
            elif S_full % sp.P:
                sp_lens = S_full
        S = x.shape[1]
        temb = F.silu(self.t_embedder(timestep, self.dtype_))
        for li, blk in enumerate(self.layers):
            m = blk.adaln(temb)                                               # [B, 4D]: scale1, gate1, scale2, gate2
            xn = fused.norm_modulate(x, weight=blk.attn_norm1, scale=m[:, 0:D], rms=True, eps=c.eps)
            qkv = blk.qkv(xn)
            fused.qk_norm_rope_(qkv, H, H, Dh, wq=blk.q_norm, wk=blk.k_norm, cos=cos, sin=sin, interleaved=True, eps=c.eps)
            q5 = qkv.view(B, S, 3, H, Dh)
            k, v = q5[:, :, 1], q5[:, :, 2]
            if past_key_values is not None:          # KV handed over by an upstream AR stage (Bagel pattern)
                pk, pv = past_key_values[li % len(past_key_values)]
                pk = pk.to(dev, x.dtype).reshape(1, -1, pk.shape[-2], Dh).expand(B, -1, -1, -1)
                pv = pv.to(dev, x.dtype).reshape(1, -1, pv.shape[-2], Dh).expand(B, -1, -1, -1)
                rep = H // pk.shape[2]
                k = torch.cat([pk.repeat_interleave(rep, 2), k], dim=1).contiguous()
                v = torch.cat([pv.repeat_interleave(rep, 2), v], dim=1).contiguous()
            if sp is not None:
                o = sp(q5, valid_len=sp_lens).reshape(B, S, H * Dh)
            else:
                o = attention(q5[:, :, 0], k, v, kv_lens=kv_lens).reshape(B, S, H * Dh)
            a = blk.out(o)
            a = fused.norm_modulate(a, weight=blk.attn_norm2, rms=True, eps=c.eps)
            x = x + torch.tanh(m[:, None, D:2 * D].float()).to(x.dtype) * a
            xn = fused.norm_modulate(x, weight=blk.ffn_norm1, scale=m[:, 2 * D:3 * D], rms=True, eps=c.eps)
            f = blk.w2(fused.silu_mul(blk.w13(xn)))
            f = fused.norm_modulate(f, weight=blk.ffn_norm2, rms=True, eps=c.eps)
            x = (x + torch.tanh(m[:, None, 3 * D:].float()).to(x.dtype) * f).contiguous()
        sc = self.final_adaln(temb)
        if sp is not None:
            x = sp.gather_rows(x, S_full, dim=1)
        out = fused.norm_modulate(x[:, :S_img].contiguous(), scale=sc, eps=1e-6)
        return self.proj_out(out)
