"""GLM-Image DiT (vllm_omni/diffusion/models/glm_image/glm_image_transformer.py:25-700).

Latents [B, C, H, W] are cut into 2x2 patches ((c, ph, pw) inside a patch) and projected; the
embedding of the AR stage's prior VQ token of every patch (zeroed where the prior is dropped for
classifier-free guidance) passes a Linear-SiLU-Linear projector and is added.  Text ("glyph")
states go through a GELU feed-forward to the model width.  Conditioning vector = timestep MLP +
MLP over the sinusoidal encodings of crop coordinates and target size.

A block modulates image and text streams with twelve vectors from one linear layer, runs ONE
attention over [text | image] with weights shared by both streams (LayerNorm without affine on
every q / k head, 2-D rotary embedding on the image rows only) and ONE shared GELU feed-forward.
In editing mode the keys / values of the condition images are cached per layer ("write") and
prepended during generation ("read").  Output: modulated LayerNorm, linear, un-patchify.

The sinusoid order inside the size embedding ([crop | target]) follows the CogView4 layer this
model derives from; diffusers is not available here to confirm it.
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


@dataclass
class GlmImageTransformerConfig:
    patch_size: int = 2
    in_channels: int = 16
    out_channels: int = 16
    num_layers: int = 30
    attention_head_dim: int = 128
    num_attention_heads: int = 32
    time_embed_dim: int = 512
    condition_dim: int = 256
    prior_vq_quantizer_codebook_size: int = 16384
    text_embed_dim: int = 1472

    @property
    def inner_dim(self) -> int:
        return self.num_attention_heads * self.attention_head_dim

    @classmethod
    def from_dict(cls, d):
        keys = set(cls.__dataclass_fields__)
        return cls(**{k: v for k, v in d.items() if k in keys})


def sinusoid(x: torch.Tensor, dim: int) -> torch.Tensor:
    """[N] -> [N, dim]: cos | sin halves (flip_sin_to_cos, no frequency shift)."""
    half = dim // 2
    a = x.float()[:, None] * torch.exp(-math.log(10000.0) * torch.arange(half, device=x.device).float() / half)[None]
    return torch.cat([a.cos(), a.sin()], dim=-1)


class _FF(nn.Module):
    """Linear, activation, Linear with diffusers' names ``net.0.proj`` / ``net.2``."""

    def __init__(self, din, inner, dout, act, dtype, device):
        super().__init__()
        self.act = act
        self.net = nn.ModuleList([nn.Module(), nn.Identity(), FusedLinear(inner, dout, dtype=dtype, device=device)])
        self.net[0].proj = FusedLinear(din, inner, dtype=dtype, device=device)

    def forward(self, x, **kw):
        h = self.net[0].proj(x.contiguous(), act="gelu_tanh" if self.act == "gelu_tanh" else ("silu" if self.act == "silu" else None))
        if self.act == "gelu":
            h = F.gelu(h.float()).to(h.dtype)
        return self.net[2](h, **kw)


class _MLP2(nn.Module):
    def __init__(self, din, dout, dtype, device):
        super().__init__()
        self.linear_1 = FusedLinear(din, dout, dtype=dtype, device=device)
        self.linear_2 = FusedLinear(dout, dout, dtype=dtype, device=device)

    def forward(self, x):
        return self.linear_2(self.linear_1(x, act="silu"))


class GlmBlock(nn.Module):
    def __init__(self, c: GlmImageTransformerConfig, dtype, device):
        super().__init__()
        D = c.inner_dim
        kw = dict(dtype=dtype, device=device)
        self.norm1 = nn.Module()
        self.norm1.linear = FusedLinear(c.time_embed_dim, 12 * D, **kw)
        self.attn1 = nn.Module()
        self.attn1.to_qkv = FusedLinear(D, 3 * D, **kw)
        self.attn1.to_out = nn.ModuleList([FusedLinear(D, D, **kw)])
        self.ff = _FF(D, 4 * D, D, "gelu_tanh", dtype, device)


class GlmLayerKV:
    """Keys / values of the condition images of one layer (image editing)."""

    def __init__(self):
        self.k = self.v = None

    def store(self, k, v):
        self.k = k if self.k is None else torch.cat([self.k, k], dim=1)
        self.v = v if self.v is None else torch.cat([self.v, v], dim=1)


class GlmImageKVCache:
    def __init__(self, num_layers: int):
        self.layers = [GlmLayerKV() for _ in range(num_layers)]
        self.mode: str | None = None          # "write" | "read" | "skip" | None

    def clear(self):
        for l in self.layers:
            l.k = l.v = None
        self.mode = None


class GlmImageTransformer2DModel(nn.Module):
    def __init__(self, cfg: GlmImageTransformerConfig | None = None, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = c = cfg or GlmImageTransformerConfig()
        self.dtype_ = dtype
        D = c.inner_dim
        kw = dict(dtype=dtype, device=device)
        self.image_projector = nn.Module()
        self.image_projector.proj = FusedLinear(c.in_channels * c.patch_size ** 2, D, **kw)
        self.glyph_projector = _FF(c.text_embed_dim, D, D, "gelu", dtype, device)
        self.prior_token_embedding = nn.Embedding(c.prior_vq_quantizer_codebook_size, D, **kw)
        self.prior_token_embedding.weight.requires_grad_(False)
        self.prior_projector = _FF(D, D, D, "silu", dtype, device)
        self.time_condition_embed = nn.Module()
        self.time_condition_embed.timestep_embedder = _MLP2(c.time_embed_dim, c.time_embed_dim, dtype, device)
        self.time_condition_embed.condition_embedder = _MLP2(4 * c.condition_dim, c.time_embed_dim, dtype, device)
        self.transformer_blocks = nn.ModuleList([GlmBlock(c, dtype, device) for _ in range(c.num_layers)])
        self.norm_out = nn.Module()
        self.norm_out.linear = FusedLinear(c.time_embed_dim, 2 * D, **kw)
        self.proj_out = FusedLinear(D, c.patch_size ** 2 * c.out_channels, **kw)
        self.block_hook = None

    # ------------------------------------------------------------------ pieces
    def patchify(self, x):
        B, C, H, W = x.shape
        p = self.cfg.patch_size
        return x.reshape(B, C, H // p, p, W // p, p).permute(0, 2, 4, 1, 3, 5).reshape(B, (H // p) * (W // p), C * p * p)

    def unpatchify(self, y, H, W):
        B = y.shape[0]
        p = self.cfg.patch_size
        return y.reshape(B, H // p, W // p, -1, p, p).permute(0, 3, 1, 4, 2, 5).reshape(B, -1, H, W)

    def rope_angles(self, h, w, device):
        Dh = self.cfg.attention_head_dim
        d = Dh // 2
        inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32)[: d // 2] / d))
        fh = torch.outer(torch.arange(h).float(), inv)[:, None].expand(h, w, -1)
        fw = torch.outer(torch.arange(w).float(), inv)[None].expand(h, w, -1)
        return torch.cat([fh, fw], dim=-1).reshape(h * w, Dh // 2).to(device)

    def condition(self, timestep, target_size, crop_coords, dtype):
        c = self.cfg
        B = timestep.shape[0]
        t = sinusoid(timestep, c.time_embed_dim).to(dtype)
        cond = torch.cat([sinusoid(crop_coords.flatten(), c.condition_dim).view(B, -1),
                          sinusoid(target_size.flatten(), c.condition_dim).view(B, -1)], dim=1).to(dtype)
        e = self.time_condition_embed
        return e.timestep_embedder(t) + e.condition_embedder(cond)

    # ------------------------------------------------------------------ forward
    def forward(self, hidden_states, encoder_hidden_states, prior_token_id, prior_token_drop, timestep, target_size,
                crop_coords, kv_cache: GlmImageKVCache | None = None, txt_seq_lens=None, **_):
        """hidden_states [B, C, H, W]; encoder_hidden_states [B, S, text_embed_dim]; prior_token_id [B, N]
        (one VQ id per patch), prior_token_drop bool [B, N]; timestep [B] (0..999); target_size / crop_coords
        [B, 2].  Returns [B, C_out, H, W]."""
        c = self.cfg
        D, H, Dh = c.inner_dim, c.num_attention_heads, c.attention_head_dim
        B, _, Hh, Ww = hidden_states.shape
        dev = hidden_states.device
        p = c.patch_size
        x = self.image_projector.proj(self.patchify(hidden_states.to(self.dtype_)).contiguous())
        txt = self.glyph_projector(encoder_hidden_states.to(self.dtype_))
        prior = self.prior_token_embedding(prior_token_id)
        prior = torch.where(prior_token_drop[..., None], torch.zeros_like(prior), prior)
        x = x + self.prior_projector(prior)
        temb = self.condition(timestep, target_size, crop_coords, self.dtype_)
        St, Si = txt.shape[1], x.shape[1]
        ang = torch.cat([torch.zeros(St, Dh // 2, device=dev), self.rope_angles(Hh // p, Ww // p, dev)])   # text rows: no rotation
        cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
        mode = kv_cache.mode if kv_cache is not None else None
        kv_lens = None
        if txt_seq_lens is not None and any(int(l) != St for l in txt_seq_lens):
            raise ValueError("GLM-Image attends text first: pad-free text rows are required (pass equal-length text states)")
        ln = lambda t: F.layer_norm(t.float(), (D,), eps=1e-5).to(t.dtype)
        for li, blk in enumerate(self.transformer_blocks):
            m = blk.norm1.linear(temb).view(B, 12, D)
            sh, csh, sc, csc, g, cg, sh2, csh2, sc2, csc2, g2, cg2 = (m[:, i, None] for i in range(12))
            u = torch.cat([ln(txt) * (1 + csc) + csh, ln(x) * (1 + sc) + sh], dim=1).contiguous()
            qkv = blk.attn1.to_qkv(u).view(B, St + Si, 3, H, Dh)
            q = F.layer_norm(qkv[:, :, 0].float(), (Dh,), eps=1e-5).to(u.dtype)
            k = F.layer_norm(qkv[:, :, 1].float(), (Dh,), eps=1e-5).to(u.dtype)
            packed = torch.stack([q, k, qkv[:, :, 2]], dim=2).reshape(B, St + Si, 3 * D).contiguous()
            fused.qk_norm_rope_(packed, H, H, Dh, cos=cos, sin=sin, interleaved=False)
            q5 = packed.view(B, St + Si, 3, H, Dh)
            kk, vv = q5[:, :, 1], q5[:, :, 2]
            if kv_cache is not None and mode == "write":
                kv_cache.layers[li].store(kk.clone(), vv.clone())
            elif kv_cache is not None and mode == "read" and kv_cache.layers[li].k is not None:
                ck, cv = kv_cache.layers[li].k, kv_cache.layers[li].v
                kk = torch.cat([ck.expand(B, -1, -1, -1), kk], dim=1).contiguous()
                vv = torch.cat([cv.expand(B, -1, -1, -1), vv], dim=1).contiguous()
            o = attention(q5[:, :, 0], kk, vv, kv_lens=kv_lens).reshape(B, St + Si, D)
            o = blk.attn1.to_out[0](o.contiguous())
            txt, x = txt + o[:, :St] * cg, x + o[:, St:] * g
            x = x + blk.ff((ln(x) * (1 + sc2) + sh2)) * g2
            txt = txt + blk.ff((ln(txt) * (1 + csc2) + csh2)) * cg2
            if self.block_hook is not None:
                self.block_hook(li, x)
        scale, shift = self.norm_out.linear(temb).chunk(2, dim=1)
        y = self.proj_out((ln(x) * (1 + scale)[:, None] + shift[:, None]).contiguous())
        return self.unpatchify(y, Hh, Ww)

    # ------------------------------------------------------------------ weights
    @torch.no_grad()
    def load_weights(self, weights) -> set:
        """diffusers names; ``attn1.to_q / to_k / to_v`` are stacked into ``attn1.to_qkv``."""
        own = dict(self.named_parameters())
        D = self.cfg.inner_dim
        loaded = set()
        for name, w in weights:
            tgt, sl = own.get(name), None
            for i, s in enumerate(("to_q", "to_k", "to_v")):
                if f".attn1.{s}." in name:
                    tgt, sl = own.get(name.replace(f".attn1.{s}.", ".attn1.to_qkv.")), (i * D, (i + 1) * D)
            if tgt is None:
                continue
            dst = tgt if sl is None else tgt[sl[0]:sl[1]]
            dst.copy_(w.to(dst.dtype).reshape(dst.shape))
            loaded.add(name)
        return loaded
