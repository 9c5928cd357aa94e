"""HunyuanImage-3 denoiser: a mixture-of-experts language model that predicts the velocity of
image latents (vllm_omni/diffusion/models/hunyuan_image_3/hunyuan_image_3_transformer.py).

Sequence of one request:  [prompt tokens] [<timestep>] [<img> x (h*w)]  (the closing <eoi> of the
reference's template is invisible to every image row under its mask and is left out).  Prompt
and <timestep> rows attend causally; image rows attend to everything before them and to every
image row (pipeline_hunyuan_image_3.py:653-673).  Positions are two-dimensional
(hunyuan_image_3_transformer.py:239-312): a text token at index i sits at (i, i), image patch
(r, c) of an h x w grid that starts at index L sits at (L + (hw - h)/2 + r, L + (hw - w)/2 + c),
i.e. the grid is centred on the diagonal stretch it occupies; even rotary pairs turn with y,
odd pairs with x, the two halves of a head are rotated against each other.  Rope comes BEFORE
the per-head RMSNorm of q and k (:1557-1563).

What is built differently from the reference:
  * After the first denoising step the reference recomputes [<timestep>, image] rows against a
    cache of the prompt's K/V that it re-assembles with ``torch.cat`` per layer and step
    (ImageKVCacheManager, :839-972).  Here every layer owns ONE [P + 1 + S, Hkv, Dh] K/V buffer per
    sequence; the prompt part is written once, each step's QKV epilogue rows are copied over the
    tail, and the attention kernel reads the buffer in place.
  * The causal part and the image part are two launches of the tcgen05 attention kernel on row
    ranges of the same buffers instead of one dense-mask SDPA over a [T, T] boolean mask.
  * Conditional and unconditional sequences share every GEMM and the grouped MoE kernel
    (rows concatenated); only attention runs per sequence.
  * The patch embedders (UNetDown / UNetUp, :2664-2796) work on the token layout directly: a
    [B, h*w, C] token matrix IS the NHWC feature map, so the 3x3 convolutions are the implicit
    GEMM of ops/conv.py with no layout change on either side of the language model.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F
from torch import nn

from ....ops import conv as C
from ....ops import fused
from ....ops.attention import attention
from ....ops.moe import MoEWorkspace, moe_forward
from ...layers.linear import FusedLinear


@dataclass
class HunyuanImage3Config:
    vocab_size: int = 133120
    hidden_size: int = 4096
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 3072
    moe_intermediate_size: int | list | None = 3072
    num_experts: int = 64
    moe_topk: int | list = 8
    num_shared_expert: int | list = 1
    use_mixed_mlp_moe: bool = True
    use_qk_norm: bool = True
    norm_topk_prob: bool = True
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    patch_size: int = 1
    patch_embed_hidden_dim: int = 1024
    latent_channels: int = 32
    vae_downsample: int = 16
    image_base_size: int = 1024
    vae: dict = field(default_factory=dict)

    @classmethod
    def from_dict(cls, d: dict | None) -> "HunyuanImage3Config":
        d = dict(d or {})
        if "attention_head_dim" in d and "head_dim" not in d:
            d["head_dim"] = d["attention_head_dim"]
        vae = d.get("vae") or {}
        if "latent_channels" in vae:
            d.setdefault("latent_channels", vae["latent_channels"])
        if "ffactor_spatial" in vae:
            d.setdefault("vae_downsample", vae["ffactor_spatial"])
        if isinstance(d.get("vae_downsample_factor"), (list, tuple)):
            d["vae_downsample"] = int(d["vae_downsample_factor"][0])
        c = cls(**{k: d[k] for k in cls.__dataclass_fields__ if k in d})
        if not c.head_dim:
            c.head_dim = c.hidden_size // c.num_attention_heads
        return c

    def per_layer(self, name: str, li: int):
        v = getattr(self, name)
        return v[li] if isinstance(v, (list, tuple)) else v


# ------------------------------------------------------------------------------------------------
# positions
# ------------------------------------------------------------------------------------------------
def rope2d_positions(seq_len: int, image_start: int | None, h: int = 0, w: int = 0) -> torch.Tensor:
    """(y, x) of every token, float64 [seq_len, 2]."""
    idx = torch.arange(seq_len, dtype=torch.float64)
    pos = torch.stack([idx, idx], dim=1)
    if image_start is not None and h * w:
        L = image_start
        by, bx = L + (w * h - h) / 2, L + (w * h - w) / 2
        ys = (by + torch.arange(h, dtype=torch.float64)).repeat_interleave(w)
        xs = (bx + torch.arange(w, dtype=torch.float64)).repeat(h)
        n = min(h * w, seq_len - L)
        pos[L:L + n, 0], pos[L:L + n, 1] = ys[:n], xs[:n]
    # the reference truncates the fractional centring offset when it builds the index tensor
    return pos.long().double()


def rope2d_cos_sin(pos: torch.Tensor, head_dim: int, theta: float = 10000.0):
    """cos / sin [T, head_dim/2] fp32: rotary pair j turns with y when j is even, x when odd, at
    frequency theta^(-2j/head_dim)."""
    assert head_dim % 4 == 0
    j = torch.arange(head_dim // 2, dtype=torch.float64)
    inv = theta ** (-2.0 * j / head_dim)
    axis = pos[:, (j.long() % 2)]                           # [T, head_dim/2]
    ang = axis * inv
    return ang.cos().float().contiguous(), ang.sin().float().contiguous()


# ------------------------------------------------------------------------------------------------
# timestep / patch embedders
# ------------------------------------------------------------------------------------------------
def sinusoid(t: torch.Tensor, dim: int, max_period: float = 10000.0) -> torch.Tensor:
    """[N] -> [N, dim]: cosines of dim/2 geometric frequencies, then the sines."""
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    a = t.float()[:, None] * freqs[None]
    return torch.cat([a.cos(), a.sin()], dim=-1)


class TimestepEmbedder(nn.Module):
    """sinusoid(256) -> Linear -> GELU -> Linear (:2535-2568); checkpoint names ``mlp.0`` / ``mlp.2``."""

    def __init__(self, hidden: int, dtype, device, freq_dim: int = 256):
        super().__init__()
        self.freq_dim = freq_dim
        self.mlp = nn.ModuleList([FusedLinear(freq_dim, hidden, dtype=dtype, device=device), nn.Identity(),
                                  FusedLinear(hidden, hidden, dtype=dtype, device=device)])

    def forward(self, t: torch.Tensor) -> torch.Tensor:
        x = sinusoid(t, self.freq_dim).to(self.mlp[0].weight.dtype)
        h = self.mlp[0](x)
        return self.mlp[2](F.gelu(h.float()).to(h.dtype))


def group_norm_tokens(x, weight, bias, groups: int = 32, eps: float = 1e-5, scale=None, shift=None, silu=True):
    """GroupNorm over a token-major feature map x [B, S, C] (statistics over S and the C/groups
    channels of a group), then ``* (1 + scale[b]) + shift[b]`` and SiLU; fp32 inside."""
    B, S, Cc = x.shape
    xf = x.float().view(B, S, groups, Cc // groups)
    mean = xf.mean(dim=(1, 3), keepdim=True)
    var = xf.var(dim=(1, 3), unbiased=False, keepdim=True)
    y = ((xf - mean) * torch.rsqrt(var + eps)).view(B, S, Cc) * weight.float() + bias.float()
    if scale is not None:
        y = y * (1.0 + scale.float()[:, None]) + shift.float()[:, None]
    if silu:
        y = F.silu(y)
    return y.to(x.dtype)


class TokenConv(nn.Module):
    """k x k convolution (k in 1, 3) over a token-major map [B, h*w, Cin] -> [B, h*w, Cout]; the
    parameter keeps the checkpoint's [Cout, Cin, k, k] layout and is packed for the implicit GEMM
    on first use."""

    def __init__(self, cin: int, cout: int, k: int, dtype, device):
        super().__init__()
        self.cin, self.cout, self.k = cin, cout, k
        self.weight = nn.Parameter(torch.empty(cout, cin, k, k, dtype=dtype, device=device).normal_(0, 0.02),
                                   requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(cout, dtype=dtype, device=device), requires_grad=False)
        self._packed = None

    def forward(self, x: torch.Tensor, h: int, w: int, residual=None) -> torch.Tensor:
        if self._packed is None or self._packed[2] != self.weight._version:
            pw, pb = C.pack_conv_weight(self.weight.data, self.bias.data, x.dtype)
            self._packed = (pw, pb, self.weight._version)
        pw, pb, _ = self._packed
        B = x.shape[0]
        ld = x.shape[-1]
        if x.is_cuda and ld % 8:                       # TMA rows start on 16 bytes
            x = F.pad(x, (0, 8 - ld % 8))
        res = residual.reshape(B, h, w, -1) if residual is not None else None
        y = C.conv2d_nhwc(x.reshape(B, h, w, -1).contiguous(), pw, pb, self.k, self.cin, residual=res)
        return y[..., :self.cout].reshape(B, h * w, self.cout) if y.shape[-1] != self.cout else y.view(B, h * w, self.cout)


class ResBlock(nn.Module):
    """GroupNorm-SiLU-conv, then GroupNorm modulated by the timestep embedding, SiLU, conv, plus a
    (1x1-projected) skip (:2571-2661).  Checkpoint names: in_layers.{0,2}, emb_layers.1,
    out_layers.{0,3}, skip_connection."""

    def __init__(self, cin: int, emb: int, cout: int, dtype, device):
        super().__init__()
        gn = lambda c: nn.GroupNorm(32, c, dtype=dtype, device=device)
        self.in_layers = nn.ModuleList([gn(cin), nn.Identity(), TokenConv(cin, cout, 3, dtype, device)])
        self.emb_layers = nn.ModuleList([nn.Identity(), FusedLinear(emb, 2 * cout, dtype=dtype, device=device)])
        self.out_layers = nn.ModuleList([gn(cout), nn.Identity(), nn.Identity(), TokenConv(cout, cout, 3, dtype, device)])
        self.skip_connection = TokenConv(cin, cout, 1, dtype, device) if cin != cout else None

    def forward(self, x: torch.Tensor, emb: torch.Tensor, h: int, w: int) -> torch.Tensor:
        n0, n1 = self.in_layers[0], self.out_layers[0]
        y = self.in_layers[2](group_norm_tokens(x, n0.weight, n0.bias, eps=n0.eps), h, w)
        e = self.emb_layers[1](F.silu(emb.float()).to(emb.dtype))
        scale, shift = e.chunk(2, dim=-1)
        y = group_norm_tokens(y, n1.weight, n1.bias, eps=n1.eps, scale=scale, shift=shift)
        skip = x if self.skip_connection is None else self.skip_connection(x, h, w)
        return self.out_layers[3](y, h, w, residual=skip.contiguous())


class UNetDown(nn.Module):
    """Latent tokens [B, h*w, C] -> tokens [B, h*w, D] (patch size 1: conv 3x3 then one ResBlock)."""

    def __init__(self, cfg: HunyuanImage3Config, dtype, device):
        super().__init__()
        assert cfg.patch_size == 1, "HunyuanImage-3 ships patch_size 1"
        hid = cfg.patch_embed_hidden_dim
        self.model = nn.ModuleList([TokenConv(cfg.latent_channels, hid, 3, dtype, device),
                                    ResBlock(hid, cfg.hidden_size, cfg.hidden_size, dtype, device)])

    def forward(self, lat: torch.Tensor, t_emb: torch.Tensor, h: int, w: int) -> torch.Tensor:
        return self.model[1](self.model[0](lat.to(t_emb.dtype), h, w), t_emb, h, w)


class UNetUp(nn.Module):
    """Tokens [B, h*w, D] -> velocity tokens [B, h*w, C]: ResBlock to the hidden width, GroupNorm-SiLU-conv."""

    def __init__(self, cfg: HunyuanImage3Config, dtype, device):
        super().__init__()
        hid = cfg.patch_embed_hidden_dim
        self.model = nn.ModuleList([
            ResBlock(cfg.hidden_size, cfg.hidden_size, hid, dtype, device),
            nn.ModuleList([nn.GroupNorm(32, hid, dtype=dtype, device=device), nn.Identity(),
                           TokenConv(hid, cfg.latent_channels, 3, dtype, device)])])

    def forward(self, x: torch.Tensor, t_emb: torch.Tensor, h: int, w: int) -> torch.Tensor:
        y = self.model[0](x, t_emb, h, w)
        n = self.model[1][0]
        return self.model[1][2](group_norm_tokens(y, n.weight, n.bias, eps=n.eps), h, w)


# ------------------------------------------------------------------------------------------------
# decoder
# ------------------------------------------------------------------------------------------------
class HunyuanDecoderLayer(nn.Module):
    def __init__(self, cfg: HunyuanImage3Config, li: int, dtype, device):
        super().__init__()
        D, H, Hkv, Dh = cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        P = lambda *s: nn.Parameter(torch.ones(*s, dtype=dtype, device=device), requires_grad=False)
        self.input_layernorm = P(D)
        self.qkv_proj = FusedLinear(D, (H + 2 * Hkv) * Dh, bias=False, dtype=dtype, device=device)
        self.q_norm = P(Dh) if cfg.use_qk_norm else None
        self.k_norm = P(Dh) if cfg.use_qk_norm else None
        self.o_proj = FusedLinear(H * Dh, D, bias=False, dtype=dtype, device=device)
        self.post_attention_layernorm = P(D)
        self.top_k = int(cfg.per_layer("moe_topk", li))
        E = cfg.num_experts
        Fm = int(cfg.per_layer("moe_intermediate_size", li) or cfg.intermediate_size)
        if E > 1:
            self.router = FusedLinear(D, E, bias=False, dtype=dtype, device=device)
            self.w13 = nn.Parameter(torch.empty(E, 2 * Fm, D, dtype=dtype, device=device).normal_(0, 0.02), requires_grad=False)
            self.w2 = nn.Parameter(torch.empty(E, D, Fm, dtype=dtype, device=device).normal_(0, 0.02), requires_grad=False)
            self.moe_ws = MoEWorkspace()
            Fs = cfg.intermediate_size * int(cfg.per_layer("num_shared_expert", li)) if cfg.use_mixed_mlp_moe else 0
        else:
            self.router = None
            Fs = cfg.intermediate_size
        self.shared_gate_up = FusedLinear(D, 2 * Fs, bias=False, dtype=dtype, device=device) if Fs else None
        self.shared_down = FusedLinear(Fs, D, bias=False, dtype=dtype, device=device) if Fs else None


@dataclass
class _Seq:
    """One sequence of the batch: P prompt rows, the <timestep> row, S image rows."""
    P: int
    S: int
    k: list = field(default_factory=list)      # per layer [P + 1 + S, Hkv, Dh]
    v: list = field(default_factory=list)

    @property
    def total(self) -> int:
        return self.P + 1 + self.S


class HunyuanImage3Model(nn.Module):
    def __init__(self, cfg: HunyuanImage3Config, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg, self.dtype_ = cfg, dtype
        self.wte = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device).normal_(0, 0.02),
                                requires_grad=False)
        self.layers = nn.ModuleList([HunyuanDecoderLayer(cfg, i, dtype, device) for i in range(cfg.num_hidden_layers)])
        self.ln_f = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype, device=device), requires_grad=False)
        self.tp_group = None
        self.tp_reduce = None
        self.ep_range = (0, cfg.num_experts)
        self.local_heads = (cfg.num_attention_heads, cfg.num_key_value_heads)

    # -- parallel layouts ------------------------------------------------------------------------
    def enable_tensor_parallel(self, group, mode: str | None = None) -> None:
        """Heads and the shared MLP's columns are sharded over the group, whole experts are dealt
        out in contiguous blocks (the reference shards heads and experts the same way,
        :1435-1470, :1335-1350); every row-parallel partial sum of a layer is finished by
        ``RowParallelReduce``."""
        from ....parallel.tensor_parallel import RowParallelReduce
        cfg = self.cfg
        n, r = group.world_size, group.rank_in_group
        if n == 1:
            return
        H, Hkv, Dh = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        assert H % n == 0 and Hkv % n == 0 and cfg.num_experts % n == 0, "heads, kv heads and experts must divide by the TP size"
        Hl, Hkvl = H // n, Hkv // n

        def relinear(old, w):
            new = FusedLinear(w.shape[1], w.shape[0], bias=False, dtype=w.dtype, device=w.device)
            new.weight.data.copy_(w)
            return new
        El = cfg.num_experts // n
        for layer in self.layers:
            w = layer.qkv_proj.weight.data
            q, k, v = w[:H * Dh], w[H * Dh:(H + Hkv) * Dh], w[(H + Hkv) * Dh:]
            layer.qkv_proj = relinear(layer.qkv_proj, torch.cat([q[r * Hl * Dh:(r + 1) * Hl * Dh],
                                                                 k[r * Hkvl * Dh:(r + 1) * Hkvl * Dh],
                                                                 v[r * Hkvl * Dh:(r + 1) * Hkvl * Dh]]).contiguous())
            layer.o_proj = relinear(layer.o_proj, layer.o_proj.weight.data[:, r * Hl * Dh:(r + 1) * Hl * Dh].contiguous())
            if layer.router is not None:
                layer.w13 = nn.Parameter(layer.w13.data[r * El:(r + 1) * El].contiguous(), requires_grad=False)
                layer.w2 = nn.Parameter(layer.w2.data[r * El:(r + 1) * El].contiguous(), requires_grad=False)
            if layer.shared_gate_up is not None:
                Fs = layer.shared_down.weight.shape[1]
                fl = Fs // n
                gu = layer.shared_gate_up.weight.data
                layer.shared_gate_up = relinear(layer.shared_gate_up, torch.cat([gu[r * fl:(r + 1) * fl],
                                                                                 gu[Fs + r * fl:Fs + (r + 1) * fl]]).contiguous())
                layer.shared_down = relinear(layer.shared_down, layer.shared_down.weight.data[:, r * fl:(r + 1) * fl].contiguous())
        self.tp_group, self.local_heads = group, (Hl, Hkvl)
        self.ep_range = (r * El, (r + 1) * El)
        self.tp_reduce = RowParallelReduce(group, mode)

    def _row_sum(self, lin: FusedLinear, a: torch.Tensor, x: torch.Tensor, cap: int) -> None:
        """x += lin(a) summed over the tensor-parallel ranks."""
        if self.tp_reduce is None:
            lin(a, residual=x, out=x)
        else:
            self.tp_reduce.linear(lin, a, residual=x, out=x, capacity=cap)

    # -- one denoising forward -------------------------------------------------------------------
    def begin(self, prompt_lens: list[int], S: int, device) -> list[_Seq]:
        """K/V buffers of a batch of sequences (one per guidance branch / prompt)."""
        Hkv, Dh = self.local_heads[1], self.cfg.head_dim
        seqs = []
        for P in prompt_lens:
            s = _Seq(P, S)
            for _ in self.layers:
                s.k.append(torch.empty(P + 1 + S, Hkv, Dh, dtype=self.dtype_, device=device))
                s.v.append(torch.empty(P + 1 + S, Hkv, Dh, dtype=self.dtype_, device=device))
            seqs.append(s)
        return seqs

    def forward(self, x: torch.Tensor, seqs: list[_Seq], cos: torch.Tensor, sin: torch.Tensor, first_step: bool) -> torch.Tensor:
        """x [T, D]: per sequence its (P + 1 + S) rows on the first step, its (1 + S) rows
        [<timestep>, image] afterwards; cos/sin [T, Dh/2] for exactly those rows.  Returns the
        hidden states [T, D] of the last layer (no final norm: the image head reads them raw,
        pipeline_hunyuan_image_3.py:963-973)."""
        cfg = self.cfg
        (H, Hkv), Dh = self.local_heads, cfg.head_dim
        T = x.shape[0]
        scale = 1.0 / math.sqrt(Dh)
        xn = torch.empty_like(x)
        attn = torch.empty(T, H * Dh, dtype=x.dtype, device=x.device)
        cap = max(64, 1 << (T - 1).bit_length())
        for li, layer in enumerate(self.layers):
            fused.norm_modulate(x, weight=layer.input_layernorm, rms=True, eps=cfg.rms_norm_eps, out=xn)
            qkv = layer.qkv_proj(xn)
            fused.qk_norm_rope_(qkv.view(1, T, -1), H, Hkv, Dh, cos=cos, sin=sin, interleaved=False)
            if layer.q_norm is not None:
                fused.qk_norm_rope_(qkv.view(1, T, -1), H, Hkv, Dh, wq=layer.q_norm, wk=layer.k_norm, eps=cfg.rms_norm_eps)
            q = qkv[:, :H * Dh].view(T, H, Dh)
            k = qkv[:, H * Dh:(H + Hkv) * Dh].view(T, Hkv, Dh)
            v = qkv[:, (H + Hkv) * Dh:].view(T, Hkv, Dh)
            o = attn.view(T, H, Dh)
            r0 = 0
            for s in seqs:
                kb, vb = s.k[li], s.v[li]
                n = s.total if first_step else 1 + s.S
                lo = 0 if first_step else s.P               # where this step's rows land in the buffers
                kb[lo:lo + n].copy_(k[r0:r0 + n])
                vb[lo:lo + n].copy_(v[r0:r0 + n])
                c = s.P + 1 - lo                            # causal rows of this step: the prompt (first step) + <timestep>
                attention(q[None, r0:r0 + c], kb[None, :s.P + 1], vb[None, :s.P + 1], scale=scale, causal=True,
                          q_offset=lo, out=o[None, r0:r0 + c])
                attention(q[None, r0 + c:r0 + n], kb[None], vb[None], scale=scale, out=o[None, r0 + c:r0 + n])
                r0 += n
            self._row_sum(layer.o_proj, attn, x, cap)
            fused.norm_modulate(x, weight=layer.post_attention_layernorm, rms=True, eps=cfg.rms_norm_eps, out=xn)
            shared = None
            if layer.shared_gate_up is not None and layer.router is not None:
                shared = fused.silu_mul(layer.shared_gate_up(xn))
            if layer.router is None:
                self._row_sum(layer.shared_down, fused.silu_mul(layer.shared_gate_up(xn)), x, cap)
                continue
            logits = layer.router(xn)
            e_lo, e_hi = self.ep_range
            renorm = cfg.norm_topk_prob and layer.top_k > 1
            if self.tp_reduce is None:
                moe_forward(xn, logits, layer.w13, layer.w2, layer.top_k, renorm, ws=layer.moe_ws, residual=x, out=x)
                if shared is not None:
                    layer.shared_down(shared, residual=x, out=x)
            else:
                part = moe_forward(xn, logits, layer.w13, layer.w2, layer.top_k, renorm, e_lo=e_lo, e_hi=e_hi, ws=layer.moe_ws)
                if shared is not None:
                    layer.shared_down(shared, residual=part, out=part)        # both partial sums ride one reduction
                self.tp_reduce(part, residual=x, out=x)
        return x

    # -- checkpoint ------------------------------------------------------------------------------
    def _split_qkv(self, w: torch.Tensor) -> torch.Tensor:
        """The checkpoint interleaves per kv head [G query heads, k, v]; ours is [all q, all k, all v]."""
        cfg = self.cfg
        H, Hkv, Dh = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        G = H // Hkv
        w = w.reshape(Hkv, G + 2, Dh, -1)
        return torch.cat([w[:, :G].reshape(H * Dh, -1), w[:, G].reshape(Hkv * Dh, -1), w[:, G + 1].reshape(Hkv * Dh, -1)])

    @staticmethod
    def _gate_first(w: torch.Tensor) -> torch.Tensor:
        """``gate_and_up_proj`` stores [up; gate]; the SiLU-mul kernels want [gate; up]."""
        half = w.shape[0] // 2
        return torch.cat([w[half:], w[:half]])

    def load_weights(self, weights, prefix: str = "model.") -> set:
        import re
        loaded = set()
        pat = re.compile(r"layers\.(\d+)\.(.+)")
        simple = {"input_layernorm.weight": "input_layernorm", "post_attention_layernorm.weight": "post_attention_layernorm",
                  "self_attn.query_layernorm.weight": "q_norm", "self_attn.key_layernorm.weight": "k_norm"}
        for name, w in weights:
            n = name[len(prefix):] if name.startswith(prefix) else name
            if n == "wte.weight":
                self.wte.data.copy_(w.to(self.wte.dtype)); loaded.add(name); continue
            if n in ("ln_f.weight", "norm.weight"):
                self.ln_f.data.copy_(w.to(self.ln_f.dtype)); loaded.add(name); continue
            m = pat.match(n)
            if not m or int(m.group(1)) >= len(self.layers):
                continue
            layer, rest = self.layers[int(m.group(1))], m.group(2)
            if rest in simple:
                p = getattr(layer, simple[rest])
                if p is not None:
                    p.data.copy_(w.to(p.dtype)); loaded.add(name)
            elif rest == "self_attn.qkv_proj.weight":
                layer.qkv_proj.weight.data.copy_(self._split_qkv(w).to(self.dtype_)); loaded.add(name)
            elif rest == "self_attn.o_proj.weight":
                layer.o_proj.weight.data.copy_(w.to(self.dtype_)); loaded.add(name)
            elif rest in ("mlp.gate.wg.weight", "mlp.gate.weight") and layer.router is not None:
                layer.router.weight.data.copy_(w.to(self.dtype_)); loaded.add(name)
            elif rest in ("mlp.shared_mlp.gate_and_up_proj.weight", "mlp.gate_and_up_proj.weight") and layer.shared_gate_up is not None:
                layer.shared_gate_up.weight.data.copy_(self._gate_first(w).to(self.dtype_)); loaded.add(name)
            elif rest in ("mlp.shared_mlp.down_proj.weight", "mlp.down_proj.weight") and layer.shared_down is not None:
                layer.shared_down.weight.data.copy_(w.to(self.dtype_)); loaded.add(name)
            else:
                me = re.match(r"mlp\.experts\.(\d+)\.(gate_and_up_proj|down_proj)\.weight", rest)
                if me and layer.router is not None and int(me.group(1)) < layer.w13.shape[0]:
                    e = int(me.group(1))
                    if me.group(2) == "down_proj":
                        layer.w2.data[e].copy_(w.to(self.dtype_))
                    else:
                        layer.w13.data[e].copy_(self._gate_first(w).to(self.dtype_))
                    loaded.add(name)
        return loaded


def reference_forward(model: HunyuanImage3Model, x: torch.Tensor, P: int, S: int, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Dense fp32 restatement of one full-sequence forward (mask, rope-then-norm, softmax
    routing), used by the tests as the oracle for the cached two-launch path."""
    cfg = model.cfg
    H, Hkv, Dh = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    T = x.shape[0]
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    mask[P + 1:, P + 1:] = True
    x = x.float()
    rms = lambda t, w: t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * w.float()

    def rope(t):
        a, b = t[..., :Dh // 2], t[..., Dh // 2:]
        c, s = cos[:, None].float(), sin[:, None].float()
        return torch.cat([a * c - b * s, b * c + a * s], dim=-1)
    for layer in model.layers:
        xn = rms(x, layer.input_layernorm)
        qkv = xn @ layer.qkv_proj.weight.float().t()
        q = rope(qkv[:, :H * Dh].view(T, H, Dh))
        k = rope(qkv[:, H * Dh:(H + Hkv) * Dh].view(T, Hkv, Dh))
        v = qkv[:, (H + Hkv) * Dh:].view(T, Hkv, Dh)
        if layer.q_norm is not None:
            q, k = rms(q, layer.q_norm), rms(k, layer.k_norm)
        k, v = k.repeat_interleave(H // Hkv, dim=1), v.repeat_interleave(H // Hkv, dim=1)
        sc = torch.einsum("thd,shd->hts", q, k) / math.sqrt(Dh)
        sc = sc.masked_fill(~mask[None], float("-inf")).softmax(-1)
        o = torch.einsum("hts,shd->thd", sc, v).reshape(T, H * Dh)
        x = x + o @ layer.o_proj.weight.float().t()
        xn = rms(x, layer.post_attention_layernorm)
        y = torch.zeros_like(x)
        if layer.router is not None:
            p = (xn @ layer.router.weight.float().t()).softmax(-1)
            wv, ids = p.topk(layer.top_k, dim=-1)
            if cfg.norm_topk_prob and layer.top_k > 1:
                wv = wv / wv.sum(-1, keepdim=True)
            Fm = layer.w2.shape[2]
            for t in range(T):
                for j in range(layer.top_k):
                    e = int(ids[t, j])
                    hh = layer.w13[e].float() @ xn[t]
                    y[t] += wv[t, j] * (layer.w2[e].float() @ (F.silu(hh[:Fm]) * hh[Fm:]))
        if layer.shared_gate_up is not None:
            hh = xn @ layer.shared_gate_up.weight.float().t()
            Fs = hh.shape[-1] // 2
            y = y + (F.silu(hh[:, :Fs]) * hh[:, Fs:]) @ layer.shared_down.weight.float().t()
        x = x + y
    return x
