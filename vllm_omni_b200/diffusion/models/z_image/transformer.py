"""Z-Image single-stream DiT (vllm_omni/diffusion/models/z_image/z_image_transformer.py:209-990).

Image latents are cut into (f, h, w) patches flattened as (pf, ph, pw, c) and embedded; caption
features go through RMSNorm + Linear.  Both token lists are padded to a multiple of 32 with learned
pad tokens.  Two "noise refiner" blocks (timestep-modulated) run on the image tokens alone, two
"context refiner" blocks (unmodulated) on the caption tokens alone; then the unified sequence
[image tokens | caption tokens] goes through the main blocks and a modulated final layer.  A block
is: RMSNorm -> (x scale) -> attention (q/k RMSNorm, 3-axis rotary with interleaved pairs) ->
RMSNorm -> (x tanh gate) -> residual; the same sandwich around a SwiGLU MLP.  Rotary positions:
caption token j at (1 + j, 0, 0), image patch (f, y, x) at (caption length + 1 + f, y, x), pad
tokens of the image list at (0, 0, 0).

Parameter names follow the checkpoint (``layers.N.attention.to_q.weight``, ``feed_forward.w1`` ...);
q/k/v and w1/w3 are stacked at load time.  The model declares a sequence-parallel plan (the
unified sequence is sharded by rows) and validates tensor-parallel divisibility like the reference
(:139-206).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ....ops import fused
from ....ops.attention import attention
from ....parallel.sp_plan import SequenceParallelInput, SequenceParallelOutput
from ...layers.linear import FusedLinear
from ..qwen_image.transformer import timestep_sinusoid

ADALN_EMBED_DIM = 256
SEQ_MULTI_OF = 32


@dataclass
class ZImageTransformerConfig:
    dim: int = 3840
    n_layers: int = 30
    n_refiner_layers: int = 2
    n_heads: int = 30
    n_kv_heads: int = 30
    norm_eps: float = 1e-5
    qk_norm: bool = True
    cap_feat_dim: int = 2560
    rope_theta: float = 256.0
    t_scale: float = 1000.0
    axes_dims: tuple = (32, 48, 48)
    axes_lens: tuple = (1024, 512, 512)
    in_channels: int = 16
    patch_size: int = 2
    f_patch_size: int = 1

    @property
    def head_dim(self) -> int:
        return self.dim // self.n_heads

    @property
    def ffn_dim(self) -> int:
        return int(self.dim / 3 * 8)

    @property
    def patch_dim(self) -> int:
        return self.f_patch_size * self.patch_size * self.patch_size * self.in_channels

    @classmethod
    def from_dict(cls, d):
        d = dict(d)
        if "all_patch_size" in d:
            d["patch_size"] = list(d.pop("all_patch_size"))[0]
        if "all_f_patch_size" in d:
            d["f_patch_size"] = list(d.pop("all_f_patch_size"))[0]
        if "axes_dims_rope" in d:
            d["axes_dims"] = d.pop("axes_dims_rope")
        keys = set(cls.__dataclass_fields__)
        return cls(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in d.items() if k in keys})


class ZBlock(nn.Module):
    def __init__(self, c: ZImageTransformerConfig, modulation: bool, dtype, device):
        super().__init__()
        D, H, Hkv, Dh = c.dim, c.n_heads, c.n_kv_heads, c.head_dim
        P = lambda *s: nn.Parameter(torch.ones(*s, dtype=dtype, device=device), requires_grad=False)
        self.modulation = modulation
        self.adaln = FusedLinear(min(D, ADALN_EMBED_DIM), 4 * D, dtype=dtype, device=device) if modulation else None
        self.attn_norm1, self.attn_norm2, self.ffn_norm1, self.ffn_norm2 = P(D), P(D), P(D), P(D)
        self.qkv = FusedLinear(D, (H + 2 * Hkv) * Dh, bias=False, dtype=dtype, device=device)
        self.q_norm, self.k_norm = (P(Dh), P(Dh)) if c.qk_norm else (None, None)
        self.out = FusedLinear(H * Dh, D, bias=False, dtype=dtype, device=device)
        self.w13 = FusedLinear(D, 2 * c.ffn_dim, bias=False, dtype=dtype, device=device)
        self.w2 = FusedLinear(c.ffn_dim, D, bias=False, dtype=dtype, device=device)


class ZImageTransformer2DModel(nn.Module):
    graph_safe_forward = True          # stateless between calls of one signature: may be replayed from a CUDA graph
    _sp_plan = {"": {"hidden_states": SequenceParallelInput(split_dim=1, expected_dims=3, auto_pad=True)},
                "proj_out": SequenceParallelOutput(gather_dim=1)}

    def __init__(self, cfg: ZImageTransformerConfig | None = None, dtype=torch.bfloat16, device=None, tp_size: int = 1):
        super().__init__()
        self.cfg = c = cfg or ZImageTransformerConfig()
        self.validate_tp(c, tp_size)
        self.dtype_ = dtype
        D, A = c.dim, min(c.dim, ADALN_EMBED_DIM)
        kw = dict(dtype=dtype, device=device)
        self.x_embedder = FusedLinear(c.patch_dim, D, **kw)
        self.cap_norm = nn.Parameter(torch.ones(c.cap_feat_dim, **kw), requires_grad=False)
        self.cap_embedder = FusedLinear(c.cap_feat_dim, D, **kw)
        self.t_mlp1 = FusedLinear(256, 1024, **kw)
        self.t_mlp2 = FusedLinear(1024, A, **kw)
        self.x_pad_token = nn.Parameter(torch.empty(1, D, **kw).normal_(0, 0.02), requires_grad=False)
        self.cap_pad_token = nn.Parameter(torch.empty(1, D, **kw).normal_(0, 0.02), requires_grad=False)
        self.noise_refiner = nn.ModuleList([ZBlock(c, True, dtype, device) for _ in range(c.n_refiner_layers)])
        self.context_refiner = nn.ModuleList([ZBlock(c, False, dtype, device) for _ in range(c.n_refiner_layers)])
        self.layers = nn.ModuleList([ZBlock(c, True, dtype, device) for _ in range(c.n_layers)])
        self.final_adaln = FusedLinear(A, D, **kw)
        self.proj_out = FusedLinear(D, c.patch_dim, **kw)
        self.block_hook = None            # observer: called as (layer index, states) after every main layer
        self.stack_hook = None            # cache backends: called once per step with a BlockStack over the main layers
        self.sp = None                   # SequenceParallelAttention when the unified sequence is sharded
        self.sp_style = "attention"
        self._tables = None
        self._layouts: dict = {}          # geometry -> position tables and masks (see _layout)

    @staticmethod
    def validate_tp(c, tp):
        if tp > 1 and (c.n_heads % tp or c.n_kv_heads % tp or c.ffn_dim % tp):
            raise ValueError(f"n_heads ({c.n_heads}), n_kv_heads ({c.n_kv_heads}) and the MLP width ({c.ffn_dim}) must be "
                             f"divisible by the tensor-parallel size {tp}")

    # ------------------------------------------------------------------ layout helpers
    def patchify(self, lat: torch.Tensor) -> torch.Tensor:
        """[B, C, H, W] (or [B, C, F, H, W]) -> [B, (f h w), (pf ph pw c)]."""
        c = self.cfg
        if lat.dim() == 4:
            lat = lat[:, :, None]
        B, C, Fr, H, W = lat.shape
        p, pf = c.patch_size, c.f_patch_size
        x = lat.reshape(B, C, Fr // pf, pf, H // p, p, W // p, p).permute(0, 2, 4, 6, 3, 5, 7, 1)
        return x.reshape(B, (Fr // pf) * (H // p) * (W // p), pf * p * p * C)

    def unpatchify(self, x: torch.Tensor, Fr: int, H: int, W: int) -> torch.Tensor:
        """[B, (f h w), (pf ph pw c)] -> [B, C, F, H, W]."""
        c = self.cfg
        p, pf = c.patch_size, c.f_patch_size
        B = x.shape[0]
        x = x.reshape(B, Fr // pf, H // p, W // p, pf, p, p, c.in_channels).permute(0, 7, 1, 4, 2, 5, 3, 6)
        return x.reshape(B, c.in_channels, Fr, H, W)

    def _rope(self, ids: torch.Tensor):
        """ids [N, 3] -> (cos, sin) [N, head_dim / 2]: per-axis angle tables, concatenated."""
        c = self.cfg
        if self._tables is None:
            self._tables = []
            for d, n in zip(c.axes_dims, c.axes_lens):
                inv = 1.0 / (c.rope_theta ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
                self._tables.append(torch.outer(torch.arange(n, dtype=torch.float64), inv).float())
        ang = torch.cat([self._tables[a].to(ids.device)[ids[:, a].long()] for a in range(len(c.axes_dims))], dim=-1)
        return ang.cos().contiguous(), ang.sin().contiguous()

    # ------------------------------------------------------------------ block
    def _block(self, blk: ZBlock, x, temb, cos, sin, positions, kv_lens, sp=None, sp_lens=None):
        c = self.cfg
        D, H, Hkv, Dh = c.dim, c.n_heads, c.n_kv_heads, c.head_dim
        B, S, _ = x.shape
        if blk.modulation:
            m = blk.adaln(temb)                                       # [B, 4D]: scale_msa, gate_msa, scale_mlp, gate_mlp
            s1, g1, s2, g2 = m[:, 0:D], m[:, D:2 * D], m[:, 2 * D:3 * D], m[:, 3 * D:]
        else:
            s1 = g1 = s2 = g2 = None
        xn = fused.norm_modulate(x, weight=blk.attn_norm1, scale=s1, rms=True, eps=c.norm_eps)
        qkv = blk.qkv(xn)
        fused.qk_norm_rope_(qkv, H, Hkv, Dh, wq=blk.q_norm, wk=blk.k_norm, cos=cos, sin=sin, interleaved=True,
                            eps=c.norm_eps, positions=positions)
        if sp is not None:
            o = sp(qkv.view(B, S, 3, H, Dh), valid_len=sp_lens).reshape(B, S, H * Dh)
        else:
            q = qkv[..., :H * Dh].view(B, S, H, Dh)
            k = qkv[..., H * Dh:(H + Hkv) * Dh].view(B, S, Hkv, Dh)
            v = qkv[..., (H + Hkv) * Dh:].view(B, S, Hkv, Dh)
            o = attention(q, k, v, kv_lens=kv_lens).reshape(B, S, H * Dh)
        a = fused.norm_modulate(blk.out(o.contiguous()), weight=blk.attn_norm2, rms=True, eps=c.norm_eps)
        x = x + (torch.tanh(g1.float()).to(x.dtype)[:, None] * a if g1 is not None else a)
        xn = fused.norm_modulate(x.contiguous(), weight=blk.ffn_norm1, scale=s2, rms=True, eps=c.norm_eps)
        f = fused.norm_modulate(blk.w2(fused.silu_mul(blk.w13(xn))), weight=blk.ffn_norm2, rms=True, eps=c.norm_eps)
        return (x + (torch.tanh(g2.float()).to(x.dtype)[:, None] * f if g2 is not None else f)).contiguous()

    # ------------------------------------------------------------------ positions
    def _layout(self, B, S_img, L, Fr, h, w, lens: tuple, dev) -> dict:
        """Everything of a forward that depends only on the shapes and caption lengths: padded lengths, position
        ids of image / caption / unified rows with their rotary tables, the rows that take the pad token and the
        rows past every caption, the key lengths.  Built on the host once per geometry and kept on the device:
        the denoising steps of a request (and a captured replay of them) reuse it."""
        key = (B, S_img, L, Fr, h, w, lens, str(dev))
        hit = self._layouts.get(key)
        if hit is not None:
            return hit
        cap_p = [n + (-n) % SEQ_MULTI_OF for n in lens]                 # caption lengths with their pad tokens
        S_x = S_img + (-S_img) % SEQ_MULTI_OF
        Lc = max(cap_p)
        grid = torch.stack(torch.meshgrid(torch.arange(Fr), torch.arange(h), torch.arange(w), indexing="ij"), -1).reshape(-1, 3)
        x_ids = torch.zeros(B, S_x, 3, dtype=torch.long)
        for b in range(B):
            x_ids[b, :S_img] = grid + torch.tensor([cap_p[b] + 1, 0, 0])
        j = torch.arange(Lc)[None, :]
        lens_t, capp_t = torch.tensor(lens)[:, None], torch.tensor(cap_p)[:, None]
        c_ids = torch.zeros(B, Lc, 3, dtype=torch.long)
        c_ids[:, :, 0] = torch.where(j < capp_t, j + 1, torch.zeros_like(j))

        def tables(ids):
            n = ids.shape[1]
            cs, sn = self._rope(ids.reshape(-1, 3).to(dev))
            pos = torch.arange(B * n, dtype=torch.int32, device=dev).view(B, n)
            return cs, sn, pos
        ragged = min(cap_p) != Lc
        lay = {"S_x": S_x, "Lc": Lc, "x": tables(x_ids), "c": tables(c_ids), "u": tables(torch.cat([x_ids, c_ids], dim=1)),
               "pad_rows": ((j >= lens_t) & (j < capp_t)).to(dev), "dead_rows": (j >= capp_t).to(dev),
               "cap_lens": torch.tensor(cap_p, dtype=torch.int32, device=dev) if ragged else None,
               "kv_lens": torch.tensor([S_x + n for n in cap_p], dtype=torch.int32, device=dev) if ragged else None}
        if len(self._layouts) < 16:           # never evicted: a captured graph may read these tensors
            self._layouts[key] = lay
        return lay

    # ------------------------------------------------------------------ forward
    def forward(self, hidden_states, encoder_hidden_states, timestep, img_shapes, txt_seq_lens=None, **_):
        """hidden_states: patchified latents [B, S_img, patch_dim]; encoder_hidden_states: caption features
        [B, L, cap_feat_dim] (rows >= txt_seq_lens[b] are padding); timestep [B] in [0, 1] (1 = clean);
        img_shapes = (f, h, w) in patches.  Returns the patch predictions [B, S_img, patch_dim]."""
        c = self.cfg
        D = c.dim
        B, S_img, L = hidden_states.shape[0], hidden_states.shape[1], encoder_hidden_states.shape[1]
        dev = hidden_states.device
        while isinstance(img_shapes[0], (list, tuple)):
            img_shapes = img_shapes[0]
        Fr, h, w = img_shapes
        lens = [int(n) for n in txt_seq_lens] if txt_seq_lens is not None else [L] * B
        lay = self._layout(B, S_img, L, Fr, h, w, tuple(lens), dev)
        S_x, Lc = lay["S_x"], lay["Lc"]

        temb = self.t_mlp2(self.t_mlp1(timestep_sinusoid(timestep, 256, c.t_scale).to(self.dtype_), act="silu"))

        # image tokens and their pad tokens
        x = self.x_embedder(hidden_states.to(self.dtype_).contiguous())
        if S_x > S_img:
            x = torch.cat([x, self.x_pad_token.to(x.dtype).expand(B, S_x - S_img, -1)], dim=1)
        # caption tokens: the last real row repeated under the pad positions is replaced by the pad token
        enc = encoder_hidden_states[:, :min(L, Lc)].to(self.dtype_).contiguous()       # rows beyond the longest caption are padding
        L = enc.shape[1]
        cap = self.cap_embedder(fused.norm_modulate(enc, weight=self.cap_norm, rms=True, eps=c.norm_eps))
        if Lc > L:
            cap = torch.cat([cap, cap.new_zeros(B, Lc - L, D)], dim=1)
        cap = torch.where(lay["pad_rows"][..., None], self.cap_pad_token.to(cap.dtype)[None], cap)
        cap = torch.where(lay["dead_rows"][..., None], torch.zeros_like(cap), cap).contiguous()

        xc, xs, xpos = lay["x"]
        for blk in self.noise_refiner:
            x = self._block(blk, x, temb, xc, xs, xpos, None)
        cc, cs_, cpos = lay["c"]
        cap_lens = lay["cap_lens"]
        for blk in self.context_refiner:
            cap = self._block(blk, cap, None, cc, cs_, cpos, cap_lens)

        u = torch.cat([x, cap], dim=1).contiguous()                      # [B, S_x + Lc, D]; rows beyond S_x + cap_p[b] are padding
        uc, us, upos = lay["u"]
        S_full = u.shape[1]
        kv_lens = lay["kv_lens"]
        sp, sp_lens = self.sp, None
        if sp is not None:
            # rows of the unified sequence are split over the SP group; padding rows are masked as keys
            u, _ = sp.shard_rows(u, dim=1)
            rows = sp.local_rows(S_full)
            pad = u.shape[1] - upos[:, rows].shape[1]
            upos = upos[:, rows]
            if pad:
                upos = torch.cat([upos, upos.new_zeros(B, pad)], dim=1)
            upos = upos.contiguous()
            sp_lens = kv_lens if kv_lens is not None else (S_full if S_full % sp.P else None)
        def run(states, a, b):
            x = states[0]
            for li in range(a, b):
                x = self._block(self.layers[li], x, temb, uc, us, upos, kv_lens, sp, sp_lens)
                if self.block_hook is not None:
                    self.block_hook(li, x)
            return (x,)
        if self.stack_hook is not None:
            from ...cache.base import BlockStack
            (u,) = self.stack_hook(BlockStack(len(self.layers), (u,), u, run))
        else:
            (u,) = run((u,), 0, len(self.layers))
        if sp is not None:
            u = sp.gather_rows(u, S_full, dim=1)
        sc = self.final_adaln(F.silu(temb))
        out = fused.norm_modulate(u[:, :S_img].contiguous(), scale=sc, eps=1e-6)
        return self.proj_out(out)

    # ------------------------------------------------------------------ weights
    def checkpoint_name_map(self) -> dict:
        """checkpoint parameter name -> (our parameter name, row slice or None)."""
        c = self.cfg
        H, Hkv, Dh, Fd = c.n_heads, c.n_kv_heads, c.head_dim, c.ffn_dim
        key = f"{c.patch_size}-{c.f_patch_size}"
        m = {}
        for wb in ("weight", "bias"):
            m[f"all_x_embedder.{key}.{wb}"] = (f"x_embedder.{wb}", None)
            m[f"all_final_layer.{key}.linear.{wb}"] = (f"proj_out.{wb}", None)
            m[f"all_final_layer.{key}.adaLN_modulation.1.{wb}"] = (f"final_adaln.{wb}", None)
            m[f"t_embedder.mlp.0.{wb}"] = (f"t_mlp1.{wb}", None)
            m[f"t_embedder.mlp.2.{wb}"] = (f"t_mlp2.{wb}", None)
            m[f"cap_embedder.1.{wb}"] = (f"cap_embedder.{wb}", None)
        m["cap_embedder.0.weight"] = ("cap_norm", None)
        m["x_pad_token"], m["cap_pad_token"] = ("x_pad_token", None), ("cap_pad_token", None)
        for group, n in (("noise_refiner", c.n_refiner_layers), ("context_refiner", c.n_refiner_layers), ("layers", c.n_layers)):
            for i in range(n):
                p = f"{group}.{i}."
                m[p + "attention.to_q.weight"] = (p + "qkv.weight", (0, H * Dh))
                m[p + "attention.to_k.weight"] = (p + "qkv.weight", (H * Dh, (H + Hkv) * Dh))
                m[p + "attention.to_v.weight"] = (p + "qkv.weight", ((H + Hkv) * Dh, (H + 2 * Hkv) * Dh))
                m[p + "attention.to_out.0.weight"] = (p + "out.weight", None)
                if c.qk_norm:
                    m[p + "attention.norm_q.weight"], m[p + "attention.norm_k.weight"] = (p + "q_norm", None), (p + "k_norm", None)
                m[p + "feed_forward.w1.weight"] = (p + "w13.weight", (0, Fd))
                m[p + "feed_forward.w3.weight"] = (p + "w13.weight", (Fd, 2 * Fd))
                m[p + "feed_forward.w2.weight"] = (p + "w2.weight", None)
                for a, b in (("attention_norm1", "attn_norm1"), ("attention_norm2", "attn_norm2"), ("ffn_norm1", "ffn_norm1"),
                             ("ffn_norm2", "ffn_norm2")):
                    m[p + a + ".weight"] = (p + b, None)
                if group != "context_refiner":
                    m[p + "adaLN_modulation.0.weight"], m[p + "adaLN_modulation.0.bias"] = (p + "adaln.weight", None), (p + "adaln.bias", None)
        return m

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        params = dict(self.named_parameters())
        nmap = self.checkpoint_name_map()
        loaded = set()
        for name, w in weights:
            if name not in nmap:
                continue
            pn, sl = nmap[name]
            dst = params[pn] if sl is None else params[pn][sl[0]:sl[1]]
            dst.copy_(w.to(dst.dtype).reshape(dst.shape))
            loaded.add(name)
        return loaded
