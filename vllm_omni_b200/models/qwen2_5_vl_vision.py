"""Vision tower of Qwen2.5-VL / Qwen2.5-Omni (the reference takes it from transformers / vLLM:
vllm_omni/model_executor/models/qwen2_5_omni/qwen2_5_omni_thinker.py, and the Qwen-Image edit
pipelines call it inside the Hugging Face text encoder, pipeline_qwen_image_edit.py).

Patches (C, t, p, p) in merge-group order -> linear patch embedding -> blocks of [RMSNorm, attention
with 2-D rotary embedding, RMSNorm, SwiGLU MLP].  Most blocks attend inside windows of
``window_size`` pixels (windows at the right / bottom edge are smaller); the blocks listed in
``fullatt_block_indexes`` attend over the whole frame.  Tokens are reordered window by window once
at the start, so every window is a contiguous run; windows become the batch dimension with a key
length per window.  A 2x2 patch merger (RMSNorm, Linear, GELU, Linear) maps to the language-model
width and the original order is restored.

Checkpoint names: ``visual.blocks.N.attn.qkv`` (Qwen2.5-VL) or ``attn.q/k/v`` (Qwen2.5-Omni),
``mlp.gate_proj/up_proj/down_proj``, ``merger.ln_q``, ``merger.mlp.0/2``, ``patch_embed.proj``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ..diffusion.layers.linear import FusedLinear
from ..ops import fused
from ..ops.attention import attention, attention_reference


@dataclass
class Qwen25VisionConfig:
    depth: int = 32
    hidden_size: int = 1280
    num_heads: int = 16
    intermediate_size: int = 3420
    patch_size: int = 14
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    in_channels: int = 3
    out_hidden_size: int = 3584
    window_size: int = 112
    fullatt_block_indexes: tuple = (7, 15, 23, 31)

    @classmethod
    def from_dict(cls, d):
        keys = set(cls.__dataclass_fields__)
        return cls(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in d.items() if k in keys})


def _mha(q, k, v, kv_lens=None):
    if q.is_cuda and q.shape[-1] in (64, 128) and q.dtype == torch.bfloat16:
        return attention(q, k, v, kv_lens=kv_lens)
    return attention_reference(q, k, v, kv_lens=kv_lens)


class VLBlock(nn.Module):
    def __init__(self, c: Qwen25VisionConfig, dtype, device):
        super().__init__()
        D = c.hidden_size
        kw = dict(dtype=dtype, device=device)
        self.heads = c.num_heads
        self.norm1 = nn.Parameter(torch.ones(D, **kw), requires_grad=False)
        self.norm2 = nn.Parameter(torch.ones(D, **kw), requires_grad=False)
        self.qkv = FusedLinear(D, 3 * D, **kw)
        self.proj = FusedLinear(D, D, **kw)
        self.gate_up = FusedLinear(D, 2 * c.intermediate_size, **kw)
        self.down = FusedLinear(c.intermediate_size, D, **kw)

    def forward(self, x, cos, sin, positions, kv_lens):           # x [B, S, D]
        B, S, D = x.shape
        H, Dh = self.heads, D // self.heads
        h = fused.norm_modulate(x, weight=self.norm1, rms=True, eps=1e-6)
        qkv = self.qkv(h)
        if qkv.is_cuda and Dh not in (64, 128):
            qkv = fused.qk_norm_rope_reference(qkv, H, H, Dh, None, None, None, None, 1 << 30, cos, sin, False, 1e-6, positions)
        else:
            fused.qk_norm_rope_(qkv, H, H, Dh, cos=cos, sin=sin, interleaved=False, positions=positions)
        q5 = qkv.view(B, S, 3, H, Dh)
        o = _mha(q5[:, :, 0], q5[:, :, 1], q5[:, :, 2], kv_lens).reshape(B, S, D)
        x = self.proj(o.contiguous(), residual=x)
        h = fused.norm_modulate(x, weight=self.norm2, rms=True, eps=1e-6)
        return self.down(fused.silu_mul(self.gate_up(h)), residual=x)


class Qwen25VisionTower(nn.Module):
    def __init__(self, cfg: Qwen25VisionConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = c = cfg
        kw = dict(dtype=dtype, device=device)
        pd = c.in_channels * c.temporal_patch_size * c.patch_size * c.patch_size
        self.patch_embed = FusedLinear(pd, c.hidden_size, bias=False, **kw)
        self.blocks = nn.ModuleList([VLBlock(c, dtype, device) for _ in range(c.depth)])
        self.group = c.hidden_size * c.spatial_merge_size ** 2
        self.ln_q = nn.Parameter(torch.ones(c.hidden_size, **kw), requires_grad=False)
        self.merge1 = FusedLinear(self.group, self.group, **kw)
        self.merge2 = FusedLinear(self.group, c.out_hidden_size, **kw)
        Dh = c.hidden_size // c.num_heads
        self.inv_freq = 1.0 / (10000.0 ** (torch.arange(0, Dh // 2, 2, dtype=torch.float32) / (Dh // 2)))

    # ------------------------------------------------------------------ layout
    def patches_from_pixels(self, pixels: torch.Tensor):
        """[T, C, H, W] frames -> (patches [t*h*w, C*tp*p*p] in merge-group order, (t, h, w))."""
        c = self.cfg
        T, C, H, W = pixels.shape
        tp, p, m = c.temporal_patch_size, c.patch_size, c.spatial_merge_size
        if T % tp:
            pixels = torch.cat([pixels, pixels[-1:].expand(tp - T % tp, -1, -1, -1)])
            T = pixels.shape[0]
        gt, gh, gw = T // tp, H // p, W // p
        x = pixels[:, :, :gh * p, :gw * p].reshape(gt, tp, C, gh // m, m, p, gw // m, m, p)
        return x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8).reshape(gt * gh * gw, -1), (gt, gh, gw)

    def _window_order(self, gt, gh, gw):
        """Permutation of the merge units (window by window) and the unit count of every window."""
        c = self.cfg
        m = c.spatial_merge_size
        ws = c.window_size // m // c.patch_size
        lh, lw = gh // m, gw // m
        idx = torch.arange(gt * lh * lw).reshape(gt, lh, lw)
        ph, pw = ws - lh % ws, ws - lw % ws                      # the reference pads a full window when the grid divides evenly
        nh, nw = (lh + ph) // ws, (lw + pw) // ws
        pad = F.pad(idx, (0, pw, 0, ph), value=-1).reshape(gt, nh, ws, nw, ws).permute(0, 1, 3, 2, 4).reshape(gt, nh * nw, ws * ws)
        counts = (pad >= 0).sum(-1).reshape(-1)
        order = pad.reshape(-1)
        return order[order >= 0], counts[counts > 0]

    # ------------------------------------------------------------------ forward
    @torch.no_grad()
    def forward_patches(self, patches: torch.Tensor, grid_thw):
        """patches: [t*h*w, C*tp*p*p] in merge-group order (the HF image processor's layout).
        Returns (merged embeddings [t*h*w/m^2, out_hidden] in the original order, merged grid)."""
        c = self.cfg
        gt, gh, gw = (int(v) for v in grid_thw)
        m = c.spatial_merge_size
        unit = m * m
        dev = patches.device
        N = gt * gh * gw
        x = self.patch_embed(patches.to(self.ln_q.dtype).contiguous())
        # (row, col) of every token in merge-group order, repeated per frame
        ys = torch.arange(gh).view(gh // m, 1, m, 1).expand(gh // m, gw // m, m, m).reshape(-1).repeat(gt)
        xs = torch.arange(gw).view(1, gw // m, 1, m).expand(gh // m, gw // m, m, m).reshape(-1).repeat(gt)
        order, counts = self._window_order(gt, gh, gw)
        tok = (order[:, None] * unit + torch.arange(unit)[None]).reshape(-1)          # token permutation
        x = x[tok.to(dev)].contiguous()
        inv = self.inv_freq
        ang = torch.cat([ys[tok].float()[:, None] * inv[None], xs[tok].float()[:, None] * inv[None]], dim=-1).to(dev)
        cos, sin = ang.cos().contiguous(), ang.sin().contiguous()                      # [N, Dh/2], window order
        # batches: whole frames, and windows padded to the largest window
        lens = (counts * unit).tolist()
        Lmax = max(lens)
        rows = torch.zeros(len(lens), Lmax, dtype=torch.long)
        valid = torch.zeros(len(lens), Lmax, dtype=torch.bool)
        o = 0
        for i, n in enumerate(lens):
            rows[i, :n] = torch.arange(o, o + n)
            valid[i, :n] = True
            o += n
        rows_d, valid_d = rows.to(dev), valid.to(dev)
        win_pos = rows_d.to(torch.int32).contiguous()
        win_lens = torch.tensor(lens, dtype=torch.int32, device=dev) if min(lens) != Lmax else None
        frame_pos = torch.arange(N, dtype=torch.int32, device=dev).view(gt, gh * gw)
        for i, blk in enumerate(self.blocks):
            if i in c.fullatt_block_indexes:
                x = blk(x.view(gt, gh * gw, -1), cos, sin, frame_pos, None).reshape(N, -1)
            else:
                y = blk(x[rows_d].contiguous(), cos, sin, win_pos, win_lens)
                x = torch.empty_like(x).index_copy_(0, rows_d[valid_d], y[valid_d])
        h = fused.norm_modulate(x.contiguous(), weight=self.ln_q, rms=True, eps=1e-6).reshape(-1, self.group)
        out = self.merge2(F.gelu(self.merge1(h.contiguous()).float()).to(h.dtype))
        return out[torch.argsort(order).to(dev)], (gt, gh // m, gw // m)

    @torch.no_grad()
    def forward(self, pixels: torch.Tensor):
        patches, grid = self.patches_from_pixels(pixels)
        out, g = self.forward_patches(patches, grid)
        return out, g, []                      # no deep-stack features in this tower

    # ------------------------------------------------------------------ weights
    @torch.no_grad()
    def load_weights(self, weights) -> set:
        """Names relative to ``visual.``."""
        D, Fi = self.cfg.hidden_size, self.cfg.intermediate_size
        simple = {"merger.ln_q.weight": self.ln_q, "merger.mlp.0.weight": self.merge1.weight, "merger.mlp.0.bias": self.merge1.bias,
                  "merger.mlp.2.weight": self.merge2.weight, "merger.mlp.2.bias": self.merge2.bias}
        loaded = set()
        for n, w in weights:
            tgt, sl = None, None
            p = n.split(".")
            if n == "patch_embed.proj.weight":
                tgt, w = self.patch_embed.weight, w.reshape(w.shape[0], -1)
            elif n in simple:
                tgt = simple[n]
            elif p[0] == "blocks":
                blk, rest = self.blocks[int(p[1])], ".".join(p[2:])
                leaf = p[-1]
                if rest in ("norm1.weight", "norm2.weight"):
                    tgt = getattr(blk, p[2])
                elif p[2] == "attn" and p[3] == "qkv":
                    tgt = getattr(blk.qkv, leaf)
                elif p[2] == "attn" and p[3] in ("q", "k", "v"):
                    i = "qkv".index(p[3])
                    tgt, sl = getattr(blk.qkv, leaf), (i * D, (i + 1) * D)
                elif p[2] == "attn" and p[3] == "proj":
                    tgt = getattr(blk.proj, leaf)
                elif p[2] == "mlp" and p[3] in ("gate_proj", "up_proj"):
                    i = 0 if p[3] == "gate_proj" else 1
                    tgt, sl = getattr(blk.gate_up, leaf), (i * Fi, (i + 1) * Fi)
                elif p[2] == "mlp" and p[3] == "down_proj":
                    tgt = getattr(blk.down, leaf)
            if tgt is None:
                continue
            dst = tgt if sl is None else tgt[sl[0]:sl[1]]
            dst.copy_(w.to(dst.dtype).reshape(dst.shape))
            loaded.add(n)
        return loaded
