"""Ovis-Image transformer (vllm_omni/diffusion/models/ovis_image/ovis_image_transformer.py:40-500):
the FLUX layout (double-stream then single-stream blocks, q/k RMSNorm, interleaved 3-axis rotary
embedding, AdaLN-Zero from the timestep alone) with gated MLPs: the double-stream feed-forwards are
SwiGLU (``net.0.proj`` emits [value | gate]) and the single-stream block's ``proj_mlp`` emits
[mlp | gate] with ``silu(gate) * mlp``.  Text states pass an RMSNorm before ``context_embedder``.
Position ids: text token i at (0, i, i), image patch (y, x) at (0, y, x).

At load time the [value | gate] halves are swapped to [gate | value], the order of this framework's
fused SiLU-multiply kernel.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn

from ....ops import fused
from ....ops.attention import attention
from ...layers.linear import FusedLinear
from ..flux.transformer import FluxTransformer2DModel, FluxTransformerConfig, SingleBlock
from ..longcat_image.transformer import longcat_rope_angles


@dataclass
class OvisTransformerConfig(FluxTransformerConfig):
    num_layers: int = 6
    num_single_layers: int = 27
    joint_attention_dim: int = 2048
    guidance_embeds: bool = False
    mlp_act: str = "swiglu"


class OvisImageTransformer2DModel(FluxTransformer2DModel):
    def __init__(self, cfg: OvisTransformerConfig | None = None, dtype=torch.bfloat16, device=None):
        cfg = cfg or OvisTransformerConfig()
        cfg.guidance_embeds, cfg.mlp_act = False, "swiglu"
        super().__init__(cfg, dtype=dtype, device=device)
        D, Fd = cfg.inner_dim, cfg.mlp_ratio * cfg.inner_dim
        kw = dict(dtype=dtype, device=device)
        self.pooled_1 = self.pooled_2 = None
        self.txt_norm_weight = nn.Parameter(torch.ones(cfg.joint_attention_dim, **kw), requires_grad=False)
        for blk in self.blocks:                                   # gated feed-forwards: [gate | value] -> F
            blk.img.mlp_up = FusedLinear(D, 2 * Fd, **kw)
            blk.txt.mlp_up = FusedLinear(D, 2 * Fd, **kw)
        for blk in self.single_blocks:                            # q | k | v | gate | mlp
            blk.linear1 = FusedLinear(D, 3 * D + 2 * Fd, **kw)

    def _cos_sin(self, h, w, txt_len, device):
        key = (h, w, txt_len, str(device))
        if key not in self._angles:
            a = longcat_rope_angles(h, w, txt_len, self.cfg.axes_dims_rope, 0, self.cfg.rope_theta, image_modality=0)
            self._angles[key] = (a.cos().contiguous().to(device), a.sin().contiguous().to(device))
        return self._angles[key]

    def single_forward(self, blk: SingleBlock, x, m3, cos, sin, kv_lens, S_img):
        cfg = self.cfg
        D, H, Hd = cfg.inner_dim, cfg.num_attention_heads, cfg.attention_head_dim
        B, S, _ = x.shape
        xn = fused.norm_modulate(x, shift=m3[:, 0:D], scale=m3[:, D:2 * D], eps=cfg.eps)
        y = blk.linear1(xn)
        qkv = y[..., :3 * D].contiguous()
        fused.qk_norm_rope_(qkv, H, H, Hd, wq=blk.norm_q, wk=blk.norm_k, cos=cos, sin=sin, interleaved=True, eps=cfg.eps)
        q5 = qkv.view(B, S, 3, H, Hd)
        o = attention(q5[:, :, 0], q5[:, :, 1], q5[:, :, 2], kv_lens=kv_lens).reshape(B, S, D)
        cat = torch.cat([o, fused.silu_mul(y[..., 3 * D:].contiguous())], dim=-1)
        blk.linear2(cat, residual=x, gate=m3[:, 2 * D:3 * D], out=x)
        return x

    def forward(self, hidden_states, encoder_hidden_states, timestep, img_shapes, txt_seq_lens=None, branch: int = 0, **_):
        enc = fused.norm_modulate(encoder_hidden_states.to(self.dtype_).contiguous(), weight=self.txt_norm_weight, rms=True,
                                  eps=1e-6)
        return super().forward(hidden_states, enc, timestep, img_shapes, pooled_projections=None, guidance=None,
                               txt_seq_lens=txt_seq_lens, branch=branch)

    # ------------------------------------------------------------------ weights
    def checkpoint_name_map(self) -> dict:
        m = {}
        for k, v in super().checkpoint_name_map().items():
            if k.startswith("time_text_embed.text_embedder") or k.startswith("time_text_embed.guidance_embedder"):
                continue
            if ".proj_mlp." in k:                                  # [mlp | gate]: twice the rows of FLUX's proj_mlp
                D, Fd = self.cfg.inner_dim, self.cfg.mlp_ratio * self.cfg.inner_dim
                v = (v[0], (3 * D, 3 * D + 2 * Fd))
            m[k.replace("time_text_embed.timestep_embedder.", "timestep_embedder.")] = v
        m["context_embedder_norm.weight"] = ("txt_norm_weight", None)
        return m

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        """[value | gate] halves of the gated projections are swapped to [gate | value]."""
        cfg = self.cfg
        D, Fd = cfg.inner_dim, cfg.mlp_ratio * cfg.inner_dim
        out = []
        for n, w in weights:
            if n.endswith((".ff.net.0.proj.weight", ".ff.net.0.proj.bias", ".ff_context.net.0.proj.weight",
                           ".ff_context.net.0.proj.bias", ".proj_mlp.weight", ".proj_mlp.bias")):
                w = torch.cat([w[Fd:], w[:Fd]], dim=0)
            out.append((n, w))
        return super().load_weights(out)
