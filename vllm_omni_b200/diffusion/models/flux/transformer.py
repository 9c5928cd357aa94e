"""FLUX-style MMDiT: double-stream blocks followed by single-stream blocks
(vllm_omni/diffusion/models/flux/flux_transformer.py).  The double-stream blocks are the same
computation as the Qwen-Image blocks and reuse that implementation (joint QKV buffer, fused
q/k-norm + RoPE, epilogue-fused gates); the single-stream block fuses its two projections
([q|k|v|mlp] in one GEMM, [attn|mlp] -> out in one GEMM with the gate and residual in the
epilogue).  Conditioning vector = timestep MLP (+ guidance MLP for distilled models) + pooled
text MLP.  Also the base of the FLUX-like members of the zoo (LongCat-Image, Ovis-Image,
FLUX.2-klein) which differ in depth, widths and text encoders.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ....ops import fused
from ....ops.attention import attention
from ...layers.linear import FusedLinear
from ..qwen_image.transformer import (QwenImageTransformer2DModel, QwenImageTransformerConfig, TimestepEmbedder,
                                      timestep_sinusoid)


@dataclass
class FluxTransformerConfig(QwenImageTransformerConfig):
    num_layers: int = 19
    num_single_layers: int = 38
    joint_attention_dim: int = 4096
    pooled_projection_dim: int = 768
    guidance_embeds: bool = True
    in_channels: int = 64
    out_channels: int = 16


def flux_rope_angles(h: int, w: int, txt_len: int, axes, theta: float = 10000.0, frames: int = 1) -> torch.Tensor:
    """Image token (y, x) -> ids (0, y, x); text tokens -> (0, 0, 0).  Image rows first."""
    def ang(idx, dim):
        inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
        return torch.outer(idx.float(), inv)
    ys = torch.arange(h).repeat_interleave(w)
    xs = torch.arange(w).repeat(h)
    # frame f (f > 0: a conditioning image appended to the image sequence) carries f on the first axis
    img = torch.cat([torch.cat([ang(torch.full((h * w,), float(f)), axes[0]), ang(ys, axes[1]), ang(xs, axes[2])], dim=-1)
                     for f in range(frames)], dim=0)
    txt = torch.zeros(txt_len, img.shape[1])
    return torch.cat([img, txt], dim=0)


class SingleBlock(nn.Module):
    def __init__(self, D, heads, head_dim, mlp_ratio, dtype, device):
        super().__init__()
        self.D, self.F = D, mlp_ratio * D
        self.linear1 = FusedLinear(D, 3 * D + self.F, dtype=dtype, device=device)      # q|k|v|mlp
        self.linear2 = FusedLinear(D + self.F, D, dtype=dtype, device=device)          # [attn|mlp] -> out
        self.norm_q = nn.Parameter(torch.ones(head_dim, dtype=dtype, device=device), requires_grad=False)
        self.norm_k = nn.Parameter(torch.ones(head_dim, dtype=dtype, device=device), requires_grad=False)


class FluxTransformer2DModel(QwenImageTransformer2DModel):
    graph_safe_forward = True          # stateless between calls of one signature: may be replayed from a CUDA graph
    def __init__(self, cfg: FluxTransformerConfig | None = None, dtype=torch.bfloat16, device=None):
        cfg = cfg or FluxTransformerConfig()
        super().__init__(cfg, dtype=dtype, device=device)
        D = cfg.inner_dim
        self.txt_norm_weight = None                       # FLUX feeds T5 states without an input norm
        self.pooled_1 = FusedLinear(cfg.pooled_projection_dim, D, dtype=dtype, device=device)
        self.pooled_2 = FusedLinear(D, D, dtype=dtype, device=device)
        self.guidance_embed = TimestepEmbedder(D, dtype, device) if cfg.guidance_embeds else None
        self.single_blocks = nn.ModuleList([SingleBlock(D, cfg.num_attention_heads, cfg.attention_head_dim,
                                                        cfg.mlp_ratio, dtype, device)
                                            for _ in range(cfg.num_single_layers)])
        self.single_mod = FusedLinear(D, cfg.num_single_layers * 3 * D, dtype=dtype, device=device)
        self._angles = {}
        self.stack_hook = None            # cache backends: called once per step with a BlockStack over double + single blocks
        self.block_hook = None            # (the Qwen-Image in-place entry is not used by this forward)

    def _cos_sin(self, h, w, txt_len, device, frames: int = 1):
        key = (h, w, txt_len, str(device), frames)
        if key not in self._angles:
            a = flux_rope_angles(h, w, txt_len, self.cfg.axes_dims_rope, self.cfg.rope_theta, frames=frames)
            self._angles[key] = (a.cos().contiguous().to(device), a.sin().contiguous().to(device))
        return self._angles[key]

    def checkpoint_name_map(self) -> dict:
        """diffusers ``FluxTransformer2DModel`` parameter name -> (our parameter name, row slice)."""
        cfg, D = self.cfg, self.cfg.inner_dim
        ren = (("img_in.", "x_embedder."), ("txt_in.", "context_embedder."), (".img_mod.1.", ".norm1.linear."),
               (".txt_mod.1.", ".norm1_context.linear."), (".img_mlp.", ".ff."), (".txt_mlp.", ".ff_context."))
        m = {}
        for k, v in super().checkpoint_name_map().items():
            if k.startswith("txt_norm"):
                continue
            for a, b in ren:
                k = k.replace(a, b) if a[0] == "." else (b + k[len(a):] if k.startswith(a) else k)
            m[k] = v
        for wb in ("weight", "bias"):
            for j in (1, 2):
                m[f"time_text_embed.text_embedder.linear_{j}.{wb}"] = (f"pooled_{j}.{wb}", None)
                if self.guidance_embed is not None:
                    m[f"time_text_embed.guidance_embedder.linear_{j}.{wb}"] = (f"guidance_embed.linear_{j}.{wb}", None)
            for i in range(cfg.num_single_layers):
                p, o = f"single_transformer_blocks.{i}.", f"single_blocks.{i}."
                m[p + f"norm.linear.{wb}"] = (f"single_mod.{wb}", (i * 3 * D, (i + 1) * 3 * D))
                for k, n in enumerate(("to_q", "to_k", "to_v")):
                    m[p + f"attn.{n}.{wb}"] = (o + f"linear1.{wb}", (k * D, (k + 1) * D))
                m[p + f"proj_mlp.{wb}"] = (o + f"linear1.{wb}", (3 * D, 3 * D + cfg.mlp_ratio * D))
                m[p + f"proj_out.{wb}"] = (o + f"linear2.{wb}", None)
        for i in range(cfg.num_single_layers):
            m[f"single_transformer_blocks.{i}.attn.norm_q.weight"] = (f"single_blocks.{i}.norm_q", None)
            m[f"single_transformer_blocks.{i}.attn.norm_k.weight"] = (f"single_blocks.{i}.norm_k", None)
        return m

    def single_forward(self, blk: SingleBlock, x, m3, cos, sin, kv_lens, S_img):
        """x: joint [B, S, D] in place; m3 [B, 3D] = shift, scale, gate.  Under tensor parallelism
        (``parallel/tensor_parallel.shard_transformer``) ``linear1`` holds this rank's heads of q, k, v and
        its slice of the MLP columns, ``linear2`` the matching input features; the partial products of
        ``linear2`` are summed across the ranks (the reference all-gathers the heads instead,
        vllm_omni/diffusion/models/flux/flux_transformer.py:230)."""
        cfg = self.cfg
        D, Hd = cfg.inner_dim, cfg.attention_head_dim
        tp = getattr(self, "tp_heads", 0)
        H = tp or cfg.num_attention_heads
        Dl = H * Hd                                  # this rank's share of the attention width
        Fl = blk.linear1.out_features - 3 * Dl       # ... and of the MLP width
        B, S, _ = x.shape
        xn = fused.norm_modulate(x, shift=m3[:, 0:D], scale=m3[:, D:2 * D], eps=cfg.eps)
        y = blk.linear1(xn)                                                    # [B,S,3Dl+Fl]
        qkv = y[..., :3 * Dl].contiguous()
        fused.qk_norm_rope_(qkv, H, H, Hd, wq=blk.norm_q, wk=blk.norm_k, cos=cos, sin=sin, interleaved=True,
                            eps=cfg.eps)
        q5 = qkv.view(B, S, 3, H, Hd)
        cat = torch.empty(B, S, Dl + Fl, dtype=x.dtype, device=x.device)
        o = attention(q5[:, :, 0], q5[:, :, 1], q5[:, :, 2], kv_lens=kv_lens)
        cat[..., :Dl] = o.reshape(B, S, Dl)
        cat[..., Dl:] = F.gelu(y[..., 3 * Dl:].float(), approximate="tanh").to(x.dtype)
        if tp:
            self.tp_reducer.linear(blk.linear2, cat, bias=blk.linear2_bias, gate=m3[:, 2 * D:3 * D], residual=x, out=x)
        else:
            blk.linear2(cat, residual=x, gate=m3[:, 2 * D:3 * D], out=x)
        return x

    def forward(self, hidden_states, encoder_hidden_states, timestep, img_shapes, pooled_projections=None,
                guidance=None, txt_seq_lens=None, branch: int = 0, **_):
        cfg, D, L = self.cfg, self.cfg.inner_dim, self.cfg.num_layers
        B, S_img, S_txt = hidden_states.shape[0], hidden_states.shape[1], encoder_hidden_states.shape[1]
        dev = hidden_states.device
        while isinstance(img_shapes[0], (list, tuple)):
            img_shapes = img_shapes[0]
        frames, h, w = img_shapes         # frames > 1: conditioning images follow the noise rows (editing)
        cos, sin = self._cos_sin(h, w, S_txt, dev, frames) if frames > 1 else self._cos_sin(h, w, S_txt, dev)
        kv_lens = None
        if txt_seq_lens is not None and any(int(l) != S_txt for l in txt_seq_lens):
            from ...graphed import device_constant
            kv_lens = device_constant([S_img + int(l) for l in txt_seq_lens], torch.int32, dev)
        img = self.img_in(hidden_states.to(self.dtype_))
        txt = self.txt_in(encoder_hidden_states.to(self.dtype_).contiguous())
        vec = self.time_embed(timestep, self.dtype_)
        if self.guidance_embed is not None:
            g = guidance if guidance is not None else torch.full((B,), 3.5, device=dev)
            vec = vec + self.guidance_embed(g, self.dtype_)          # the embedder scales by 1000 itself
        if pooled_projections is not None:
            vec = vec + self.pooled_2(self.pooled_1(pooled_projections.to(self.dtype_), act="silu"))
        sv = F.silu(vec)
        mods = self.mod(sv).view(B, L, 2, 6 * D)
        ws = self._workspace(B, S_img, S_txt, dev)
        m3 = self.single_mod(sv).view(B, cfg.num_single_layers, 3 * D)
        Ls = cfg.num_single_layers

        def run(states, a, b):
            """Blocks a..b-1 of [double blocks | single blocks] on the (image, text) streams."""
            im, tx = states
            for i in range(a, min(b, L)):
                self.block_forward(i, im, tx, mods, cos, sin, kv_lens, ws)
            if b > L and max(a, L) < b:
                x = torch.cat([im, tx], dim=1).contiguous()
                for j in range(max(a, L) - L, b - L):
                    self.single_forward(self.single_blocks[j], x, m3[:, j], cos, sin, kv_lens, S_img)
                im, tx = x[:, :S_img].contiguous(), x[:, S_img:].contiguous()
            return (im, tx)
        if self.stack_hook is not None:
            from ...cache.base import BlockStack
            m0 = mods[:, 0, 0]
            probe = fused.norm_modulate(img, shift=m0[:, 0:D], scale=m0[:, D:2 * D], eps=cfg.eps)
            img, txt = self.stack_hook(BlockStack(L + Ls, (img, txt), probe, run, branch=branch))
        else:
            img, txt = run((img, txt), 0, L + Ls)
        ss = self.norm_out(sv)
        out = fused.norm_modulate(img.contiguous(), shift=ss[:, D:], scale=ss[:, :D], eps=cfg.eps)
        return self.proj_out(out)
