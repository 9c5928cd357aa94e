"""BAGEL's mixture-of-transformers language model used as the image denoiser
(vllm_omni/diffusion/models/bagel/bagel_transformer.py:253-720, 831-1504).

A Qwen2-style decoder (q/k/v biases, per-head q/k RMS norm, GQA) with TWO sets of weights per layer:
the understanding set (checkpoint names as in Qwen2) processes text tokens, the generation set
(``*_moe_gen``) processes the noisy VAE latent tokens.  One image is the query sequence
``<|vision_start|> latent tokens <|vision_end|>``; all of its tokens share ONE rotary position (the
length of the context so far), attend to each other without a causal mask and to the key/value
cache of the context (the prompt, prefilled here in understanding mode or handed over by the AR
stage).  Latent tokens enter as ``vae2llm(x_t) + time embedding + 2-D sin-cos position embedding`` and
leave through ``llm2vae`` as the flow velocity.

Layout here: the latent rows come first and the two marker rows last, so that the generation weights
run on a contiguous block and the fused q/k-norm + rotary kernel can switch norm weights at one row
index; attention is order-free.  Only the two marker rows of the embedding table are kept for
generation, the full table only when the prompt is prefilled in this stage.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch
import torch.nn.functional as F
from torch import nn

from ....ops import fused
from ....ops.attention import attention, attention_reference
from ...layers.linear import FusedLinear
from ..qwen_image.transformer import timestep_sinusoid


@dataclass
class BagelMoTConfig:
    vocab_size: int = 152064
    hidden_size: int = 3584
    num_hidden_layers: int = 28
    num_attention_heads: int = 28
    num_key_value_heads: int = 4
    intermediate_size: int = 18944
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    latent_patch_size: int = 2
    max_latent_size: int = 64
    z_channels: int = 16
    vae_downsample: int = 8
    timestep_shift: float = 3.0
    start_of_image: int = 151652            # <|vision_start|>
    end_of_image: int = 151653              # <|vision_end|>
    bos_token_id: int = 151644              # <|im_start|>
    eos_token_id: int = 151645              # <|im_end|>
    keep_embedding_table: bool = True       # False: only the marker rows are loaded (context always arrives as KV)

    @classmethod
    def from_dict(cls, d: dict) -> "BagelMoTConfig":
        d = dict(d)
        llm = d.pop("llm_config", None) or {}
        vae = d.pop("vae_config", None) or {}
        merged = {**llm, **d}
        if "z_channels" in vae:
            merged.setdefault("z_channels", vae["z_channels"])
        if "downsample" in vae:
            merged.setdefault("vae_downsample", vae["downsample"])
        keys = set(cls.__dataclass_fields__)
        return cls(**{k: v for k, v in merged.items() if k in keys})

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def patch_latent_dim(self) -> int:
        return self.latent_patch_size ** 2 * self.z_channels

    @property
    def latent_downsample(self) -> int:
        return self.vae_downsample * self.latent_patch_size


def sincos_2d_table(dim: int, grid: int) -> torch.Tensor:
    """[grid * grid, dim]: per axis [sin | cos] of the coordinate over ``dim / 4`` frequencies; the first
    half of the channels encodes the COLUMN, the second half the row (row-major positions)."""
    def axis(pos):
        omega = 1.0 / 10000 ** (np.arange(dim // 4, dtype=np.float64) / (dim / 4.0))
        out = np.einsum("m,d->md", pos.reshape(-1), omega)
        return np.concatenate([np.sin(out), np.cos(out)], axis=1)
    gw, gh = np.meshgrid(np.arange(grid, dtype=np.float32), np.arange(grid, dtype=np.float32))
    return torch.from_numpy(np.concatenate([axis(gw), axis(gh)], axis=1)).float()


def latent_position_ids(h: int, w: int, max_side: int) -> torch.Tensor:
    return (torch.arange(h)[:, None] * max_side + torch.arange(w)[None]).flatten()


def _mha(q, k, v, causal=False):
    off = k.shape[1] - q.shape[1]                      # queries are the last rows of the key sequence
    if q.is_cuda and q.shape[-1] in (64, 128) and q.dtype == torch.bfloat16:
        return attention(q, k, v, causal=causal, q_offset=off)
    return attention_reference(q, k, v, causal=causal, q_offset=off)


class _Stream(nn.Module):
    """One weight set of a layer (understanding or generation)."""

    def __init__(self, c: BagelMoTConfig, dtype, device):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        D, H, Hkv, Dh = c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim
        P = lambda n: nn.Parameter(torch.ones(n, **kw), requires_grad=False)
        self.input_layernorm, self.post_attention_layernorm = P(D), P(D)
        self.qkv = FusedLinear(D, (H + 2 * Hkv) * Dh, bias=True, **kw)
        self.q_norm, self.k_norm = P(Dh), P(Dh)
        self.o = FusedLinear(H * Dh, D, bias=False, **kw)
        self.gate_up = FusedLinear(D, 2 * c.intermediate_size, bias=False, **kw)
        self.down = FusedLinear(c.intermediate_size, D, bias=False, **kw)


class MoTLayer(nn.Module):
    def __init__(self, c: BagelMoTConfig, dtype, device):
        super().__init__()
        self.und, self.gen = _Stream(c, dtype, device), _Stream(c, dtype, device)


class BagelMoT(nn.Module):
    def __init__(self, cfg: BagelMoTConfig | None = None, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = c = cfg or BagelMoTConfig()
        self.dtype_ = dtype
        kw = dict(dtype=dtype, device=device)
        D = c.hidden_size
        rows = c.vocab_size if c.keep_embedding_table else 2
        self.embed_tokens = nn.Parameter(torch.empty(rows, D, **kw).normal_(0, 0.02), requires_grad=False)
        self.layers = nn.ModuleList([MoTLayer(c, dtype, device) for _ in range(c.num_hidden_layers)])
        self.norm = nn.Parameter(torch.ones(D, **kw), requires_grad=False)
        self.norm_moe_gen = nn.Parameter(torch.ones(D, **kw), requires_grad=False)
        self.time_1, self.time_2 = FusedLinear(256, D, **kw), FusedLinear(D, D, **kw)
        self.vae2llm, self.llm2vae = FusedLinear(c.patch_latent_dim, D, **kw), FusedLinear(D, c.patch_latent_dim, **kw)
        self.latent_pos_embed = nn.Parameter(sincos_2d_table(D, c.max_latent_size).to(**kw), requires_grad=False)
        self.inv_freq = 1.0 / (c.rope_theta ** (torch.arange(0, c.head_dim, 2, dtype=torch.float32) / c.head_dim))
        self.stack_hook = None            # cache backends: called per velocity evaluation with a BlockStack over the layers

    # ------------------------------------------------------------------ helpers
    def _embed(self, ids: torch.Tensor) -> torch.Tensor:
        if self.cfg.keep_embedding_table:
            return self.embed_tokens[ids]
        c = self.cfg
        idx = torch.where(ids == c.start_of_image, 0, 1)
        if not bool(((ids == c.start_of_image) | (ids == c.end_of_image)).all()):
            raise ValueError("this model keeps only the image marker rows of the embedding table")
        return self.embed_tokens[idx]

    def _cos_sin(self, positions: torch.Tensor):
        ang = positions.float()[:, None] * self.inv_freq.to(positions.device)[None]
        return ang.cos().contiguous(), ang.sin().contiguous()

    def _qkv_heads(self, qkv):
        c = self.cfg
        H, Hkv, Dh = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        B, S = qkv.shape[:2]
        q = qkv[..., :H * Dh].view(B, S, H, Dh)
        k = qkv[..., H * Dh:(H + Hkv) * Dh].view(B, S, Hkv, Dh)
        v = qkv[..., (H + Hkv) * Dh:].view(B, S, Hkv, Dh)
        return q, k, v

    def _norm_rope(self, qkv, cos, sin, wq, wk, wq_alt=None, wk_alt=None, s_alt=1 << 30):
        c = self.cfg
        H, Hkv, Dh = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        if qkv.is_cuda and Dh not in (64, 128):
            return fused.qk_norm_rope_reference(qkv, H, Hkv, Dh, wq, wk, wq_alt, wk_alt, s_alt, cos, sin, False, c.rms_norm_eps)
        return fused.qk_norm_rope_(qkv, H, Hkv, Dh, wq=wq, wk=wk, wq_alt=wq_alt, wk_alt=wk_alt, s_alt=s_alt, cos=cos, sin=sin,
                                   interleaved=False, eps=c.rms_norm_eps)

    def _attend(self, q, k, v, past, li, causal):
        c = self.cfg
        if past is not None and past[li] is not None and past[li][0].shape[0] > 0:
            pk, pv = past[li]
            B = q.shape[0]
            k = torch.cat([pk.to(k)[None].expand(B, -1, -1, -1), k], dim=1)
            v = torch.cat([pv.to(v)[None].expand(B, -1, -1, -1), v], dim=1)
        rep = c.num_attention_heads // c.num_key_value_heads
        if rep > 1:
            k, v = k.repeat_interleave(rep, dim=2), v.repeat_interleave(rep, dim=2)
        return _mha(q.contiguous(), k.contiguous(), v.contiguous(), causal=causal)

    # ------------------------------------------------------------------ understanding mode: prefill of text
    @torch.no_grad()
    def prefill_text(self, ids: torch.Tensor, past=None, start_position: int = 0):
        """ids [L] appended to the context ``past`` (list of (k, v) [T, Hkv, Dh] per layer or None) at
        rotary positions start_position..; returns the grown context."""
        c = self.cfg
        eps = c.rms_norm_eps
        x = self._embed(ids)[None].to(self.dtype_)                       # [1, L, D]
        L = ids.shape[0]
        cos, sin = self._cos_sin(torch.arange(start_position, start_position + L, device=ids.device))
        out = []
        for li, layer in enumerate(self.layers):
            s = layer.und
            h = fused.norm_modulate(x, weight=s.input_layernorm, rms=True, eps=eps)
            qkv = self._norm_rope(s.qkv(h), cos, sin, s.q_norm, s.k_norm)
            q, k, v = self._qkv_heads(qkv)
            pk, pv = (past[li] if past is not None and past[li] is not None else (k[0, :0], v[0, :0]))
            out.append((torch.cat([pk.to(k), k[0]], 0), torch.cat([pv.to(v), v[0]], 0)))
            o = self._attend(q, k, v, past, li, causal=True).reshape(1, L, -1)
            x = s.o(o.contiguous(), residual=x)
            h = fused.norm_modulate(x, weight=s.post_attention_layernorm, rms=True, eps=eps)
            x = s.down(fused.silu_mul(s.gate_up(h)), residual=x)
        return out

    def _gen_layer(self, li, x, N, cos, sin, past, collect=None):
        """One layer in generation mode: latent rows [0, N) on the generation weights, the other rows on the
        understanding weights, full attention among them and over the context.  ``collect``: a list that
        receives this layer's (k, v) of the rows (batch 0), for callers that grow the context."""
        c = self.cfg
        eps = c.rms_norm_eps
        B, S = x.shape[0], x.shape[1]
        layer = self.layers[li]
        g, u = layer.gen, layer.und
        if N == 0:                                       # understanding rows only (vision-tower tokens + markers)
            ht = fused.norm_modulate(x.contiguous(), weight=u.input_layernorm, rms=True, eps=eps)
            qkv = self._norm_rope(u.qkv(ht).contiguous(), cos, sin, u.q_norm, u.k_norm)
        else:
            hv = fused.norm_modulate(x[:, :N].contiguous(), weight=g.input_layernorm, rms=True, eps=eps)
            ht = fused.norm_modulate(x[:, N:].contiguous(), weight=u.input_layernorm, rms=True, eps=eps)
            qkv = torch.cat([g.qkv(hv), u.qkv(ht)], dim=1).contiguous()
            qkv = self._norm_rope(qkv, cos, sin, g.q_norm, g.k_norm, u.q_norm, u.k_norm, N)
        q, k, v = self._qkv_heads(qkv)
        if collect is not None:
            collect.append((k[0].clone(), v[0].clone()))
        o = self._attend(q, k, v, past, li, causal=False).reshape(B, S, -1)
        if N == 0:
            xt = u.o(o.contiguous(), residual=x.contiguous())
            ht = fused.norm_modulate(xt, weight=u.post_attention_layernorm, rms=True, eps=eps)
            return u.down(fused.silu_mul(u.gate_up(ht)), residual=xt)
        xv = g.o(o[:, :N].contiguous(), residual=x[:, :N].contiguous())
        xt = u.o(o[:, N:].contiguous(), residual=x[:, N:].contiguous())
        hv = fused.norm_modulate(xv, weight=g.post_attention_layernorm, rms=True, eps=eps)
        ht = fused.norm_modulate(xt, weight=u.post_attention_layernorm, rms=True, eps=eps)
        xv = g.down(fused.silu_mul(g.gate_up(hv)), residual=xv)
        xt = u.down(fused.silu_mul(u.gate_up(ht)), residual=xt)
        return torch.cat([xv, xt], dim=1)

    # ------------------------------------------------------------------ editing context: images in front of the prompt
    def _latent_rows(self, x_t, t, grid):
        """Latent tokens -> language-model rows: projection + timestep embedding + 2-D position table."""
        c = self.cfg
        dt = self.dtype_
        B = x_t.shape[0]
        h, w = grid
        pos_ids = latent_position_ids(h, w, c.max_latent_size).to(x_t.device)
        tt = t.reshape(-1).expand(B) if t.numel() == 1 else t.reshape(-1)
        temb = self.time_2(self.time_1(timestep_sinusoid(tt, 256, scale=1.0).to(dt), act="silu"))
        return self.vae2llm(x_t.to(dt).contiguous()) + temb[:, None] + self.latent_pos_embed[pos_ids][None]

    @torch.no_grad()
    def _append_block(self, x, n_gen, past, position):
        """Run ``x`` [1, S, D] (first ``n_gen`` rows on the generation weights) against the context, all rows at
        rotary position ``position`` with full attention among them, and return the context grown by the
        block's K/V (bagel_transformer.py:1012-1071, :1136-1189: ``update_past_key_values`` with
        ``is_causal=False``)."""
        S = x.shape[1]
        cos, sin = self._cos_sin(torch.full((S,), int(position), device=x.device))
        grown = []
        for li in range(len(self.layers)):
            got = []
            x = self._gen_layer(li, x, n_gen, cos, sin, past, collect=got)
            k, v = got[0]
            pk, pv = (past[li] if past is not None and past[li] is not None else (k[:0], v[:0]))
            grown.append((torch.cat([pk.to(k), k], 0), torch.cat([pv.to(v), v], 0)))
        return grown

    @torch.no_grad()
    def prefill_image_latents(self, latent_tokens: torch.Tensor, grid, past=None, position: int = 0):
        """A clean image as context: its VAE latents [N, patch_latent_dim] at timestep 0 between the two image
        markers (latent rows on the generation weights, markers on the understanding weights).  Occupies ONE
        rotary position; returns the grown context."""
        c = self.cfg
        dev = latent_tokens.device
        lat = self._latent_rows(latent_tokens[None], torch.zeros(1, device=dev), grid)
        marks = self._embed(torch.tensor([c.start_of_image, c.end_of_image], device=dev)).to(self.dtype_)
        x = torch.cat([lat, marks[None]], dim=1).contiguous()
        return self._append_block(x, latent_tokens.shape[0], past, position)

    @torch.no_grad()
    def prefill_vision_tokens(self, tokens: torch.Tensor, past=None, position: int = 0):
        """Vision-tower tokens [Nv, D] (already in the language model's width, position table added) between
        the image markers, all on the understanding weights, at one rotary position."""
        c = self.cfg
        marks = self._embed(torch.tensor([c.start_of_image, c.end_of_image], device=tokens.device)).to(self.dtype_)
        x = torch.cat([tokens.to(self.dtype_), marks], dim=0)[None].contiguous()
        return self._append_block(x, 0, past, position)

    # ------------------------------------------------------------------ generation mode: one velocity evaluation
    @torch.no_grad()
    def flow(self, x_t: torch.Tensor, t: torch.Tensor, grid, past=None, position: int = 0, branch: int = 0) -> torch.Tensor:
        """x_t [B, N, patch_latent_dim] (N = h * w latent tokens), t [B] in [0, 1], grid (h, w), context
        ``past`` of length ``position`` rows (or any length, with the image placed at rotary position
        ``position``) -> velocity [B, N, patch_latent_dim]."""
        c = self.cfg
        eps, D = c.rms_norm_eps, c.hidden_size
        dt = self.dtype_
        B, N, _ = x_t.shape
        dev = x_t.device
        h, w = grid
        lat = self._latent_rows(x_t, t, grid)
        marks = self._embed(torch.tensor([c.start_of_image, c.end_of_image], device=dev)).to(dt)
        x = torch.cat([lat, marks[None].expand(B, -1, -1)], dim=1).contiguous()            # [B, N + 2, D]
        S = N + 2
        cos, sin = self._cos_sin(torch.full((S,), int(position), device=dev))
        def run(states, a, b):
            x = states[0]
            for li in range(a, b):
                x = self._gen_layer(li, x, N, cos, sin, past)
            return (x,)
        if self.stack_hook is not None:
            from ...cache.base import BlockStack
            (x,) = self.stack_hook(BlockStack(len(self.layers), (x,), x[:, :N], run, branch=branch))
        else:
            (x,) = run((x,), 0, len(self.layers))
        out = fused.norm_modulate(x[:, :N].contiguous(), weight=self.norm_moe_gen, rms=True, eps=eps)
        return self.llm2vae(out)

    # ------------------------------------------------------------------ weights
    @torch.no_grad()
    def load_weights(self, weights) -> set:
        """Names of the published checkpoint: ``language_model.model.layers.N.*`` (with ``*_moe_gen``
        twins), ``language_model.model.{embed_tokens,norm,norm_moe_gen}``, ``time_embedder.mlp.0|2``,
        ``vae2llm``, ``llm2vae``, ``latent_pos_embed.pos_embed``.  Other tensors (vision tower, connector,
        ``lm_head``) are ignored."""
        c = self.cfg
        H, Hkv, Dh, Fi = c.num_attention_heads, c.num_key_value_heads, c.head_dim, c.intermediate_size
        qo = {"q_proj": (0, H * Dh), "k_proj": (H * Dh, (H + Hkv) * Dh), "v_proj": ((H + Hkv) * Dh, (H + 2 * Hkv) * Dh)}
        top = {"time_embedder.mlp.0": self.time_1, "time_embedder.mlp.2": self.time_2, "vae2llm": self.vae2llm, "llm2vae": self.llm2vae}
        loaded = set()
        for full, w in weights:
            n = full
            for pre in ("module.", "bagel.", "language_model.", "model."):
                if n.startswith(pre):
                    n = n[len(pre):]
            tgt, sl = None, None
            stem, _, leaf = n.rpartition(".")
            if stem in top:
                tgt = getattr(top[stem], leaf, None)
            elif n == "latent_pos_embed.pos_embed":
                tgt = self.latent_pos_embed
            elif n == "embed_tokens.weight":
                if c.keep_embedding_table:
                    tgt = self.embed_tokens
                else:
                    self.embed_tokens.copy_(w[[c.start_of_image, c.end_of_image]].to(self.embed_tokens.dtype))
                    loaded.add(full)
                    continue
            elif n == "norm.weight":
                tgt = self.norm
            elif n == "norm_moe_gen.weight":
                tgt = self.norm_moe_gen
            elif n.startswith("layers."):
                p = n.split(".")
                layer = self.layers[int(p[1])]
                gen = "_moe_gen" in n
                s = layer.gen if gen else layer.und
                rest = ".".join(p[2:]).replace("_moe_gen", "")
                r = rest.split(".")
                if r[0] == "self_attn" and r[1] in qo:
                    tgt, sl = getattr(s.qkv, r[2]), qo[r[1]]
                elif r[0] == "self_attn" and r[1] == "o_proj":
                    tgt = getattr(s.o, r[2])
                elif r[0] == "self_attn" and r[1] in ("q_norm", "k_norm"):
                    tgt = getattr(s, r[1])
                elif r[0] == "mlp" and r[1] in ("gate_proj", "up_proj"):
                    i = 0 if r[1] == "gate_proj" else 1
                    tgt, sl = s.gate_up.weight, (i * Fi, (i + 1) * Fi)
                elif r[0] == "mlp" and r[1] == "down_proj":
                    tgt = s.down.weight
                elif r[0] in ("input_layernorm", "post_attention_layernorm"):
                    tgt = getattr(s, r[0])
            if tgt is None:
                continue
            dst = tgt if sl is None else tgt[sl[0]:sl[1]]
            dst.copy_(w.to(dst.dtype).reshape(dst.shape))
            loaded.add(full)
        return loaded
