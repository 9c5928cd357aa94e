"""Stable Diffusion 3 MMDiT (vllm_omni/diffusion/models/sd3/sd3_transformer.py; diffusers
``SD3Transformer2DModel``): 2x2 patch embedding plus a centre-cropped 2-D sin/cos position table,
joint-attention blocks over [image | text] WITHOUT rotary embedding (q/k RMSNorm only in the 3.5
checkpoints), AdaLN-Zero modulation from timestep + pooled text vector, a last block whose text
stream is only normalised (``context_pre_only``), AdaLN-continuous output layer.

The joint block is the same computation as the Qwen-Image / FLUX double-stream block, so the fused
implementation (stacked modulation GEMM, shared QKV buffer, epilogue-fused gates) is reused with
the rotary tables switched off.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ....ops import fused
from ...layers.linear import FusedLinear
from ..flux.transformer import FluxTransformer2DModel, FluxTransformerConfig


@dataclass
class SD3TransformerConfig(FluxTransformerConfig):
    num_layers: int = 24
    num_single_layers: int = 0
    attention_head_dim: int = 64
    num_attention_heads: int = 24
    joint_attention_dim: int = 4096
    pooled_projection_dim: int = 2048
    guidance_embeds: bool = False
    in_channels: int = 64                  # 2x2 patches of the 16-channel latent
    out_channels: int = 16
    pos_embed_max_size: int = 192
    qk_norm: str | None = None             # "rms_norm" in the 3.5 checkpoints
    dual_attention_layers: tuple = ()
    eps: float = 1e-6

    @classmethod
    def from_dict(cls, d):
        d = dict(d)
        if d.get("in_channels") == 16 and "patch_size" in d:          # diffusers counts latent channels, not patch width
            d["in_channels"] = 16 * int(d["patch_size"]) ** 2
        keys = set(cls.__dataclass_fields__)
        return cls(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in d.items() if k in keys})


def sincos_2d(dim: int, grid: int, base_size: int, interpolation_scale: float = 1.0) -> torch.Tensor:
    """[grid*grid, dim] table: first half encodes the column (x), second half the row (y) coordinate,
    each as [sin | cos] over dim/4 frequencies; coordinates are scaled by base_size / grid."""
    pos = torch.arange(grid, dtype=torch.float64) / (grid / base_size) / interpolation_scale
    omega = 1.0 / (10000 ** (torch.arange(dim // 4, dtype=torch.float64) / (dim / 4)))
    def enc(p):
        a = p[:, None] * omega[None]
        return torch.cat([a.sin(), a.cos()], dim=1)
    ys, xs = torch.meshgrid(pos, pos, indexing="ij")
    return torch.cat([enc(xs.reshape(-1)), enc(ys.reshape(-1))], dim=1).float()


class SD3Transformer2DModel(FluxTransformer2DModel):
    def __init__(self, cfg: SD3TransformerConfig | None = None, dtype=torch.bfloat16, device=None, sample_size: int = 128):
        cfg = cfg or SD3TransformerConfig()
        if cfg.dual_attention_layers:
            raise NotImplementedError("the second image-only attention of the SD3.5-medium blocks is not built")
        super().__init__(cfg, dtype=dtype, device=device)
        D = cfg.inner_dim
        table = sincos_2d(D, cfg.pos_embed_max_size, sample_size // 2)
        self.pos_table = nn.Parameter(table.to(dtype=dtype, device=device), requires_grad=False)
        if cfg.qk_norm is None:
            for blk in self.blocks:
                blk.img.norm_q = blk.img.norm_k = blk.txt.norm_q = blk.txt.norm_k = None

    def _pos(self, h, w):
        M = self.cfg.pos_embed_max_size
        if h > M or w > M:
            raise ValueError(f"latent grid {h}x{w} exceeds the position table ({M}x{M})")
        t, l = (M - h) // 2, (M - w) // 2
        return self.pos_table.view(M, M, -1)[t:t + h, l:l + w].reshape(h * w, -1)

    def forward(self, hidden_states, encoder_hidden_states, timestep, img_shapes, pooled_projections=None,
                txt_seq_lens=None, **_):
        cfg, D, L = self.cfg, self.cfg.inner_dim, self.cfg.num_layers
        B, S_img, S_txt = hidden_states.shape[0], hidden_states.shape[1], encoder_hidden_states.shape[1]
        dev = hidden_states.device
        while isinstance(img_shapes[0], (list, tuple)):
            img_shapes = img_shapes[0]
        _, h, w = img_shapes
        kv_lens = None
        if txt_seq_lens is not None and any(int(l) != S_txt for l in txt_seq_lens):
            kv_lens = torch.tensor([S_img + int(l) for l in txt_seq_lens], dtype=torch.int32, device=dev)
        img = (self.img_in(hidden_states.to(self.dtype_)) + self._pos(h, w)[None]).contiguous()
        txt = self.txt_in(encoder_hidden_states.to(self.dtype_).contiguous())
        vec = self.time_embed(timestep, self.dtype_)
        if pooled_projections is not None:
            vec = vec + self.pooled_2(self.pooled_1(pooled_projections.to(self.dtype_), act="silu"))
        sv = F.silu(vec)
        mods = self.mod(sv).view(B, L, 2, 6 * D)
        ws = self._workspace(B, S_img, S_txt, dev)
        def run(states, a, b):
            for i in range(a, b):
                self.block_forward(i, img, txt, mods, None, None, kv_lens, ws)   # in place; no rotary embedding
            return (img, txt)
        if self.stack_hook is not None:
            from ...cache.base import BlockStack
            m0 = mods[:, 0, 0]
            probe = fused.norm_modulate(img, shift=m0[:, 0:D], scale=m0[:, D:2 * D], eps=cfg.eps)
            self.stack_hook(BlockStack(L, (img, txt), probe, run))
        else:
            run((img, txt), 0, L)
        ss = self.norm_out(sv)
        out = fused.norm_modulate(img, shift=ss[:, D:], scale=ss[:, :D], eps=cfg.eps)
        return self.proj_out(out)

    def checkpoint_name_map(self) -> dict:
        """diffusers ``SD3Transformer2DModel`` parameter name -> (our parameter name, row slice)."""
        cfg, D, L = self.cfg, self.cfg.inner_dim, self.cfg.num_layers
        m = {}
        last = f"transformer_blocks.{L - 1}."
        for k, v in super().checkpoint_name_map().items():
            if k.startswith("x_embedder."):
                k = "pos_embed.proj." + k[len("x_embedder."):]
            if k.startswith(last) and (".ff_context." in k or ".attn.to_add_out." in k or ".norm1_context." in k):
                continue                                              # the last block's text stream ends after attention
            if cfg.qk_norm is None and ".attn.norm_" in k:
                continue
            m[k] = v
        # last block: AdaLN-continuous on the text stream, rows [scale | shift] -> our [shift, scale, ...] slots
        r0 = ((L - 1) * 2 + 1) * 6 * D
        for wb in ("weight", "bias"):
            m[last + f"norm1_context.linear.{wb}#scale"] = (f"mod.{wb}", (r0 + D, r0 + 2 * D))
            m[last + f"norm1_context.linear.{wb}#shift"] = (f"mod.{wb}", (r0, r0 + D))
        m["pos_embed.pos_embed"] = ("pos_table", None)
        return m

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        L, D = self.cfg.num_layers, self.cfg.inner_dim
        split = f"transformer_blocks.{L - 1}.norm1_context.linear."
        expanded, origin = [], {}
        for n, w in weights:
            if n.startswith(split):
                for tag, rows in (("#scale", slice(0, D)), ("#shift", slice(D, 2 * D))):
                    expanded.append((n + tag, w[rows]))
                    origin[n + tag] = n
            elif n == "pos_embed.proj.weight":
                expanded.append((n, w.reshape(w.shape[0], -1)))       # conv [D, C, 2, 2] -> linear over (c, ph, pw)
            elif n in ("proj_out.weight", "proj_out.bias"):
                # the checkpoint emits a patch as (ph, pw, c); the pipeline's packed layout is (c, ph, pw)
                C = self.cfg.out_channels
                pp = w.shape[0] // C
                expanded.append((n, w.reshape(pp, C, *w.shape[1:]).transpose(0, 1).reshape(w.shape)))
            else:
                expanded.append((n, w))
        loaded = super().load_weights(expanded)
        return {origin.get(n, n) for n in loaded}
