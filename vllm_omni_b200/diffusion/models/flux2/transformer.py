"""FLUX.2 transformer, the denoiser of FLUX.2-klein
(vllm_omni/diffusion/models/flux2_klein/flux2_klein_transformer.py:45-768).

What sets it apart from FLUX.1: no biases anywhere; ONE modulation per step shared by all
double-stream blocks (one for the image stream, one for the text stream) and one shared by all
single-stream blocks, so the AdaLN parameters are computed once per step rather than per block;
SwiGLU feed-forwards (ratio 3); single-stream blocks whose input GEMM emits [q | k | v | gate | up] and
whose output GEMM takes [attention | SwiGLU]; a four-axis rotary embedding (theta 2000) driven by
position ids of the image AND the text tokens; no pooled text vector.

B200 mapping: per block the image and text projections write into one joint [image rows | text rows]
qkv buffer; q/k RMS norm (per-stream weights) and the interleaved rotary turn are one in-place kernel
over that buffer; attention runs on the joint sequence; gates and residuals ride in the epilogue of
the output GEMMs.  The reference orders the joint sequence text-first; attention does not care about
the order as long as every token keeps its own rotary angles, which is how the tables are built here.

Checkpoint names (diffusers ``Flux2Transformer2DModel``): ``transformer_blocks.N.attn.{to_q,to_k,to_v,
add_q_proj,add_k_proj,add_v_proj,to_out.0,to_add_out,norm_q,norm_k,norm_added_q,norm_added_k}``,
``ff|ff_context.{linear_in,linear_out}``, ``single_transformer_blocks.N.attn.{to_qkv_mlp_proj,to_out,
norm_q,norm_k}``, ``double_stream_modulation_img|txt.linear``, ``single_stream_modulation.linear``,
``time_guidance_embed.{timestep_embedder,guidance_embedder}.linear_1|2``, ``x_embedder``,
``context_embedder``, ``norm_out.linear``, ``proj_out``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ....ops import fused
from ....ops.attention import attention, attention_reference
from ...layers.linear import FusedLinear
from ..qwen_image.transformer import timestep_sinusoid


@dataclass
class Flux2TransformerConfig:
    patch_size: int = 1
    in_channels: int = 128
    out_channels: int | None = None
    num_layers: int = 8
    num_single_layers: int = 48
    attention_head_dim: int = 128
    num_attention_heads: int = 48
    joint_attention_dim: int = 15360
    timestep_guidance_channels: int = 256
    mlp_ratio: float = 3.0
    axes_dims_rope: tuple = (32, 32, 32, 32)
    rope_theta: float = 2000.0
    eps: float = 1e-6
    guidance_embeds: bool = True

    @classmethod
    def from_dict(cls, d: dict) -> "Flux2TransformerConfig":
        keys = set(cls.__dataclass_fields__)
        return cls(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in d.items() if k in keys})

    @property
    def inner_dim(self) -> int:
        return self.num_attention_heads * self.attention_head_dim


def flux2_rope_angles(ids: torch.Tensor, axes, theta: float) -> torch.Tensor:
    """ids [S, n_axes] -> angles [S, sum(axes) / 2]: axis a contributes ``axes[a] / 2`` frequencies of its coordinate."""
    out = []
    for a, dim in enumerate(axes):
        inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float64, device=ids.device) / dim))
        out.append(ids[:, a].double()[:, None] * inv[None])
    return torch.cat(out, dim=-1).float()


def image_ids(h: int, w: int, t: int = 0) -> torch.Tensor:
    """Position ids (t, y, x, 0) of an h x w token grid in row-major order."""
    ys = torch.arange(h).repeat_interleave(w)
    xs = torch.arange(w).repeat(h)
    return torch.stack([torch.full_like(ys, t), ys, xs, torch.zeros_like(ys)], dim=-1)


def text_ids(n: int) -> torch.Tensor:
    """Position ids (0, 0, 0, l) of n text tokens."""
    z = torch.zeros(n, dtype=torch.long)
    return torch.stack([z, z, z, torch.arange(n)], dim=-1)


def _mha(q, k, v, kv_lens=None):
    if q.is_cuda and q.shape[-1] in (64, 128) and q.dtype == torch.bfloat16:
        return attention(q, k, v, kv_lens=kv_lens)
    return attention_reference(q, k, v, kv_lens=kv_lens)


class _TimeMLP(nn.Module):
    def __init__(self, cin, dim, dtype, device):
        super().__init__()
        self.linear_1 = FusedLinear(cin, dim, bias=False, dtype=dtype, device=device)
        self.linear_2 = FusedLinear(dim, dim, bias=False, dtype=dtype, device=device)

    def forward(self, t, cin, dtype):
        return self.linear_2(self.linear_1(timestep_sinusoid(t, cin).to(dtype), act="silu"))


class DoubleBlock(nn.Module):
    def __init__(self, c: Flux2TransformerConfig, dtype, device):
        super().__init__()
        kw = dict(bias=False, dtype=dtype, device=device)
        D, Dh, Fi = c.inner_dim, c.attention_head_dim, int(c.inner_dim * c.mlp_ratio)
        P = lambda: nn.Parameter(torch.ones(Dh, dtype=dtype, device=device), requires_grad=False)
        self.to_qkv, self.add_qkv = FusedLinear(D, 3 * D, **kw), FusedLinear(D, 3 * D, **kw)
        self.norm_q, self.norm_k, self.norm_added_q, self.norm_added_k = P(), P(), P(), P()
        self.to_out, self.to_add_out = FusedLinear(D, D, **kw), FusedLinear(D, D, **kw)
        self.ff_in, self.ff_out = FusedLinear(D, 2 * Fi, **kw), FusedLinear(Fi, D, **kw)
        self.ffc_in, self.ffc_out = FusedLinear(D, 2 * Fi, **kw), FusedLinear(Fi, D, **kw)


class SingleBlock(nn.Module):
    def __init__(self, c: Flux2TransformerConfig, dtype, device):
        super().__init__()
        kw = dict(bias=False, dtype=dtype, device=device)
        D, Dh, Fi = c.inner_dim, c.attention_head_dim, int(c.inner_dim * c.mlp_ratio)
        self.qkv_mlp = FusedLinear(D, 3 * D + 2 * Fi, **kw)
        self.out = FusedLinear(D + Fi, D, **kw)
        self.norm_q = nn.Parameter(torch.ones(Dh, dtype=dtype, device=device), requires_grad=False)
        self.norm_k = nn.Parameter(torch.ones(Dh, dtype=dtype, device=device), requires_grad=False)


class Flux2Transformer2DModel(nn.Module):
    graph_safe_forward = True          # stateless between calls of one signature: may be replayed from a CUDA graph
    def __init__(self, cfg: Flux2TransformerConfig | None = None, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = c = cfg or Flux2TransformerConfig()
        self.dtype_ = dtype
        kw = dict(bias=False, dtype=dtype, device=device)
        D = c.inner_dim
        self.out_channels = c.out_channels or c.in_channels
        self.time_embed = _TimeMLP(c.timestep_guidance_channels, D, dtype, device)
        self.guidance_embed = _TimeMLP(c.timestep_guidance_channels, D, dtype, device) if c.guidance_embeds else None
        self.mod_img, self.mod_txt, self.mod_single = FusedLinear(D, 6 * D, **kw), FusedLinear(D, 6 * D, **kw), FusedLinear(D, 3 * D, **kw)
        self.x_embedder = FusedLinear(c.in_channels, D, **kw)
        self.context_embedder = FusedLinear(c.joint_attention_dim, D, **kw)
        self.blocks = nn.ModuleList([DoubleBlock(c, dtype, device) for _ in range(c.num_layers)])
        self.single_blocks = nn.ModuleList([SingleBlock(c, dtype, device) for _ in range(c.num_single_layers)])
        self.norm_out = FusedLinear(D, 2 * D, **kw)
        self.proj_out = FusedLinear(D, c.patch_size * c.patch_size * self.out_channels, **kw)
        self._angles: dict = {}
        self.stack_hook = None            # cache backends: called once per step with a BlockStack over double + single blocks

    # ------------------------------------------------------------------ rotary tables
    def cos_sin(self, img_ids: torch.Tensor, txt_ids: torch.Tensor, device):
        """Tables for the joint [image | text] order, cached per id tensors."""
        key = (tuple(img_ids.shape), tuple(txt_ids.shape), int(img_ids.sum()), int(txt_ids.sum()), int((img_ids * img_ids).sum()),
               str(device))
        hit = self._angles.get(key)
        if hit is None:
            ang = flux2_rope_angles(torch.cat([img_ids, txt_ids], 0).cpu(), self.cfg.axes_dims_rope, self.cfg.rope_theta)
            hit = (ang.cos().contiguous().to(device), ang.sin().contiguous().to(device))
            self._angles = {key: hit}
        return hit

    # ------------------------------------------------------------------ blocks
    def _double(self, blk: DoubleBlock, img, txt, mi, mt, cos, sin, kv_lens):
        c = self.cfg
        D, H, Dh = c.inner_dim, c.num_attention_heads, c.attention_head_dim
        B, Si, St = img.shape[0], img.shape[1], txt.shape[1]
        qkv = torch.empty(B, Si + St, 3 * D, dtype=img.dtype, device=img.device)
        qkv[:, :Si] = blk.to_qkv(fused.norm_modulate(img, shift=mi[:, 0:D], scale=mi[:, D:2 * D], eps=c.eps))
        qkv[:, Si:] = blk.add_qkv(fused.norm_modulate(txt, shift=mt[:, 0:D], scale=mt[:, D:2 * D], eps=c.eps))
        if qkv.is_cuda and Dh not in (64, 128):
            qkv = fused.qk_norm_rope_reference(qkv, H, H, Dh, blk.norm_q, blk.norm_k, blk.norm_added_q, blk.norm_added_k, Si,
                                               cos, sin, True, c.eps)
        else:
            fused.qk_norm_rope_(qkv, H, H, Dh, wq=blk.norm_q, wk=blk.norm_k, wq_alt=blk.norm_added_q, wk_alt=blk.norm_added_k,
                                s_alt=Si, cos=cos, sin=sin, interleaved=True, eps=c.eps)
        q5 = qkv.view(B, Si + St, 3, H, Dh)
        o = _mha(q5[:, :, 0], q5[:, :, 1], q5[:, :, 2], kv_lens).reshape(B, Si + St, D)
        img = blk.to_out(o[:, :Si].contiguous(), residual=img, gate=mi[:, 2 * D:3 * D])
        txt = blk.to_add_out(o[:, Si:].contiguous(), residual=txt, gate=mt[:, 2 * D:3 * D])
        h = fused.norm_modulate(img, shift=mi[:, 3 * D:4 * D], scale=mi[:, 4 * D:5 * D], eps=c.eps)
        img = blk.ff_out(fused.silu_mul(blk.ff_in(h)), residual=img, gate=mi[:, 5 * D:6 * D])
        h = fused.norm_modulate(txt, shift=mt[:, 3 * D:4 * D], scale=mt[:, 4 * D:5 * D], eps=c.eps)
        txt = blk.ffc_out(fused.silu_mul(blk.ffc_in(h)), residual=txt, gate=mt[:, 5 * D:6 * D])
        return img, txt

    def _single(self, blk: SingleBlock, x, ms, cos, sin, kv_lens):
        c = self.cfg
        D, H, Dh = c.inner_dim, c.num_attention_heads, c.attention_head_dim
        B, S, _ = x.shape
        y = blk.qkv_mlp(fused.norm_modulate(x, shift=ms[:, 0:D], scale=ms[:, D:2 * D], eps=c.eps))
        qkv = y[..., :3 * D].contiguous()
        if qkv.is_cuda and Dh not in (64, 128):
            qkv = fused.qk_norm_rope_reference(qkv, H, H, Dh, blk.norm_q, blk.norm_k, None, None, 1 << 30, cos, sin, True, c.eps)
        else:
            fused.qk_norm_rope_(qkv, H, H, Dh, wq=blk.norm_q, wk=blk.norm_k, cos=cos, sin=sin, interleaved=True, eps=c.eps)
        q5 = qkv.view(B, S, 3, H, Dh)
        Fi = (y.shape[-1] - 3 * D) // 2
        cat = torch.empty(B, S, D + Fi, dtype=x.dtype, device=x.device)
        cat[..., :D] = _mha(q5[:, :, 0], q5[:, :, 1], q5[:, :, 2], kv_lens).reshape(B, S, D)
        cat[..., D:] = fused.silu_mul(y[..., 3 * D:].contiguous())
        return blk.out(cat, residual=x, gate=ms[:, 2 * D:3 * D])

    # ------------------------------------------------------------------ forward
    @torch.no_grad()
    def forward(self, hidden_states, encoder_hidden_states, timestep, img_ids, txt_ids, guidance=None, txt_seq_lens=None,
                branch: int = 0, **_):
        """hidden_states [B, S_img, C], encoder_hidden_states [B, S_txt, J], timestep [B] in [0, 1],
        img_ids [S_img, 4], txt_ids [S_txt, 4] -> [B, S_img, patch^2 * out_channels]."""
        c = self.cfg
        D = c.inner_dim
        dt = self.dtype_
        B, Si, St = hidden_states.shape[0], hidden_states.shape[1], encoder_hidden_states.shape[1]
        dev = hidden_states.device
        img_ids = img_ids[0] if img_ids.dim() == 3 else img_ids
        txt_ids = txt_ids[0] if txt_ids.dim() == 3 else txt_ids
        cos, sin = self.cos_sin(img_ids, txt_ids, dev)
        kv_lens = None
        if txt_seq_lens is not None and any(int(l) != St for l in txt_seq_lens):
            from ...graphed import device_constant
            kv_lens = device_constant([Si + int(l) for l in txt_seq_lens], torch.int32, dev)
        t = timestep.reshape(-1).expand(B) if timestep.numel() == 1 else timestep.reshape(-1)
        temb = self.time_embed(t, c.timestep_guidance_channels, dt)
        if guidance is not None and self.guidance_embed is not None:
            temb = temb + self.guidance_embed(guidance.reshape(-1).expand(B) if guidance.numel() == 1 else guidance.reshape(-1),
                                              c.timestep_guidance_channels, dt)
        sv = F.silu(temb)
        mi, mt, ms = self.mod_img(sv), self.mod_txt(sv), self.mod_single(sv)
        img = self.x_embedder(hidden_states.to(dt).contiguous())
        txt = self.context_embedder(encoder_hidden_states.to(dt).contiguous())
        L, Ls = len(self.blocks), len(self.single_blocks)

        def run(states, a, b):
            im, tx = states
            for i in range(a, min(b, L)):
                im, tx = self._double(self.blocks[i], im, tx, mi, mt, cos, sin, kv_lens)
            if b > L and max(a, L) < b:
                x = torch.cat([im, tx], dim=1).contiguous()
                for j in range(max(a, L) - L, b - L):
                    x = self._single(self.single_blocks[j], x, ms, cos, sin, kv_lens)
                im, tx = x[:, :Si].contiguous(), x[:, Si:].contiguous()
            return (im, tx)
        if self.stack_hook is not None:
            from ...cache.base import BlockStack
            probe = fused.norm_modulate(img, shift=mi[:, 0:D], scale=mi[:, D:2 * D], eps=c.eps)
            img, txt = self.stack_hook(BlockStack(L + Ls, (img, txt), probe, run, branch=branch))
        else:
            img, txt = run((img, txt), 0, L + Ls)
        ss = self.norm_out(sv)                                   # scale | shift
        out = fused.norm_modulate(img.contiguous(), shift=ss[:, D:], scale=ss[:, :D], eps=c.eps)
        return self.proj_out(out)

    # ------------------------------------------------------------------ weights
    def checkpoint_name_map(self) -> dict:
        """diffusers parameter name -> (our parameter name, row slice or None)."""
        c, D = self.cfg, self.cfg.inner_dim
        m = {"x_embedder.weight": ("x_embedder.weight", None), "context_embedder.weight": ("context_embedder.weight", None),
             "double_stream_modulation_img.linear.weight": ("mod_img.weight", None),
             "double_stream_modulation_txt.linear.weight": ("mod_txt.weight", None),
             "single_stream_modulation.linear.weight": ("mod_single.weight", None),
             "norm_out.linear.weight": ("norm_out.weight", None), "proj_out.weight": ("proj_out.weight", None)}
        for j in (1, 2):
            m[f"time_guidance_embed.timestep_embedder.linear_{j}.weight"] = (f"time_embed.linear_{j}.weight", None)
            if self.guidance_embed is not None:
                m[f"time_guidance_embed.guidance_embedder.linear_{j}.weight"] = (f"guidance_embed.linear_{j}.weight", None)
        for i in range(c.num_layers):
            p, o = f"transformer_blocks.{i}.", f"blocks.{i}."
            for k, n in enumerate(("to_q", "to_k", "to_v")):
                m[p + f"attn.{n}.weight"] = (o + "to_qkv.weight", (k * D, (k + 1) * D))
            for k, n in enumerate(("add_q_proj", "add_k_proj", "add_v_proj")):
                m[p + f"attn.{n}.weight"] = (o + "add_qkv.weight", (k * D, (k + 1) * D))
            for n in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
                m[p + f"attn.{n}.weight"] = (o + n, None)
            m[p + "attn.to_out.0.weight"] = (o + "to_out.weight", None)
            m[p + "attn.to_add_out.weight"] = (o + "to_add_out.weight", None)
            m[p + "ff.linear_in.weight"], m[p + "ff.linear_out.weight"] = (o + "ff_in.weight", None), (o + "ff_out.weight", None)
            m[p + "ff_context.linear_in.weight"] = (o + "ffc_in.weight", None)
            m[p + "ff_context.linear_out.weight"] = (o + "ffc_out.weight", None)
        for i in range(c.num_single_layers):
            p, o = f"single_transformer_blocks.{i}.", f"single_blocks.{i}."
            m[p + "attn.to_qkv_mlp_proj.weight"] = (o + "qkv_mlp.weight", None)
            m[p + "attn.to_out.weight"] = (o + "out.weight", None)
            m[p + "attn.norm_q.weight"], m[p + "attn.norm_k.weight"] = (o + "norm_q", None), (o + "norm_k", None)
        return m

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        params = dict(self.named_parameters())
        nm = self.checkpoint_name_map()
        loaded = set()
        for n, w in weights:
            n2 = n.replace("to_qkvkv_mlp_proj", "to_qkv_mlp_proj")      # a misspelling found in some exports
            if n2 not in nm:
                continue
            pn, sl = nm[n2]
            dst = params[pn] if sl is None else params[pn][sl[0]:sl[1]]
            dst.copy_(w.to(dst.dtype).reshape(dst.shape))
            loaded.add(n)
        return loaded
