"""Vision side of BAGEL's editing context: a SigLIP encoder run NaViT-style (patches of one image
at native aspect ratio, position table looked up by (row, column)), the two-layer connector into the
language model's width and the frozen sin-cos position table that is added after it
(vllm_omni/diffusion/models/bagel/pipeline_bagel.py:122-150 ``SiglipNaViTWrapper``,
bagel_transformer.py:58-76 ``MLPconnector``, :806-821 ``PositionEmbedding``, :1136-1189).

The reference calls the HF ``SiglipVisionModel``'s encoder with a block-diagonal mask over the packed
patches of all images; one image per call needs no mask.  Checkpoint names:
``vit_model.vision_model.embeddings.{patch_embedding,position_embedding}``,
``vit_model.vision_model.encoder.layers.N.{layer_norm1,self_attn.{q,k,v,out}_proj,layer_norm2,mlp.fc1,mlp.fc2}``
(the encoder's output is used WITHOUT ``post_layernorm``), ``connector.fc1|fc2``, ``vit_pos_embed.pos_embed``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ....ops.attention import attention, attention_reference
from ...layers.linear import FusedLinear


@dataclass
class BagelVitConfig:
    hidden_size: int = 1152
    intermediate_size: int = 4304
    num_hidden_layers: int = 26
    num_attention_heads: int = 16
    patch_size: int = 14
    max_patches_per_side: int = 70
    layer_norm_eps: float = 1e-6

    @classmethod
    def from_dict(cls, d: dict | None) -> "BagelVitConfig":
        d = d or {}
        return cls(**{k: d[k] for k in cls.__dataclass_fields__ if k in d})


def patchify_pixels(img: torch.Tensor, p: int) -> torch.Tensor:
    """[3, H, W] -> [H/p * W/p, 3*p*p], each patch flattened (channel, row, column) as a Conv2d kernel is."""
    C, H, W = img.shape
    x = img.reshape(C, H // p, p, W // p, p).permute(1, 3, 0, 2, 4)
    return x.reshape((H // p) * (W // p), C * p * p)


def flat_position_ids(h: int, w: int, max_side: int) -> torch.Tensor:
    return (torch.arange(h)[:, None] * max_side + torch.arange(w)[None]).flatten()


class _VitLayer(nn.Module):
    def __init__(self, c: BagelVitConfig, dtype, device):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        D = c.hidden_size
        self.layer_norm1 = nn.LayerNorm(D, eps=c.layer_norm_eps, **kw)
        self.layer_norm2 = nn.LayerNorm(D, eps=c.layer_norm_eps, **kw)
        self.qkv = FusedLinear(D, 3 * D, **kw)             # q_proj | k_proj | v_proj rows
        self.out_proj = FusedLinear(D, D, **kw)
        self.fc1, self.fc2 = FusedLinear(D, c.intermediate_size, **kw), FusedLinear(c.intermediate_size, D, **kw)


class BagelVisionTower(nn.Module):
    def __init__(self, cfg: BagelVitConfig, llm_width: int, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = c = cfg
        kw = dict(dtype=dtype, device=device)
        D = c.hidden_size
        self.patch_embedding = FusedLinear(3 * c.patch_size ** 2, D, **kw)
        self.position_embedding = nn.Parameter(torch.zeros(c.max_patches_per_side ** 2, D, **kw).normal_(0, 0.02),
                                               requires_grad=False)
        self.layers = nn.ModuleList([_VitLayer(c, dtype, device) for _ in range(c.num_hidden_layers)])
        self.connector_fc1 = FusedLinear(D, llm_width, **kw)
        self.connector_fc2 = FusedLinear(llm_width, llm_width, **kw)
        from .mot import sincos_2d_table
        self.vit_pos_embed = nn.Parameter(sincos_2d_table(llm_width, c.max_patches_per_side).to(**kw), requires_grad=False)

    @torch.no_grad()
    def forward(self, pixels: torch.Tensor) -> torch.Tensor:
        """pixels [3, H, W] in [-1, 1], H and W multiples of the patch size -> [H/p * W/p, llm_width]."""
        c = self.cfg
        dt = self.patch_embedding.weight.dtype
        h, w = pixels.shape[1] // c.patch_size, pixels.shape[2] // c.patch_size
        if max(h, w) > c.max_patches_per_side:
            raise ValueError(f"{h}x{w} patches exceed the tower's {c.max_patches_per_side} per side")
        ids = flat_position_ids(h, w, c.max_patches_per_side).to(pixels.device)
        x = self.patch_embedding(patchify_pixels(pixels.to(dt), c.patch_size).contiguous()) + self.position_embedding[ids]
        H = c.num_attention_heads
        Dh = c.hidden_size // H
        N = x.shape[0]
        for L in self.layers:
            y = F.layer_norm(x, (c.hidden_size,), L.layer_norm1.weight, L.layer_norm1.bias, c.layer_norm_eps)
            q, k, v = L.qkv(y).view(1, N, 3, H, Dh).unbind(2)
            if x.is_cuda and Dh in (64, 128) and x.dtype == torch.bfloat16:
                o = attention(q, k, v)
            else:
                o = attention_reference(q, k, v)
            x = L.out_proj(o.reshape(N, -1).contiguous(), residual=x)
            y = F.layer_norm(x, (c.hidden_size,), L.layer_norm2.weight, L.layer_norm2.bias, c.layer_norm_eps)
            x = L.fc2(L.fc1(y, act="gelu_tanh"), residual=x)
        x = self.connector_fc2(self.connector_fc1(x, act="gelu_tanh"))
        return x + self.vit_pos_embed[ids]

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        c = self.cfg
        D = c.hidden_size
        loaded = set()
        qkv_rows = {"q_proj": 0, "k_proj": 1, "v_proj": 2}
        for full, w in weights:
            n = full
            for pre in ("module.", "bagel."):
                if n.startswith(pre):
                    n = n[len(pre):]
            tgt = None
            if n.startswith("vit_model."):
                m = n[len("vit_model."):]
                if m.startswith("vision_model."):
                    m = m[len("vision_model."):]
                p = m.split(".")
                if m.startswith("embeddings.patch_embedding."):
                    tgt = getattr(self.patch_embedding, p[-1])
                elif m == "embeddings.position_embedding.weight":
                    tgt = self.position_embedding
                elif m.startswith("encoder.layers.") and int(p[2]) < len(self.layers):
                    L = self.layers[int(p[2])]
                    if p[3] == "self_attn" and p[4] in qkv_rows:
                        i = qkv_rows[p[4]]
                        tgt = getattr(L.qkv, p[5])[i * D:(i + 1) * D]
                    elif p[3] == "self_attn" and p[4] == "out_proj":
                        tgt = getattr(L.out_proj, p[5])
                    elif p[3] in ("layer_norm1", "layer_norm2"):
                        tgt = getattr(getattr(L, p[3]), p[4])
                    elif p[3] == "mlp" and p[4] in ("fc1", "fc2"):
                        tgt = getattr(getattr(L, p[4]), p[5])
            elif n.startswith("connector.fc1."):
                tgt = getattr(self.connector_fc1, n.rsplit(".", 1)[1])
            elif n.startswith("connector.fc2."):
                tgt = getattr(self.connector_fc2, n.rsplit(".", 1)[1])
            elif n == "vit_pos_embed.pos_embed":
                tgt = self.vit_pos_embed
            if tgt is None:
                continue
            tgt.copy_(w.to(tgt.dtype).reshape(tgt.shape))
            loaded.add(full)
        return loaded
