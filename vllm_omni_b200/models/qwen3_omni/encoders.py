"""Audio and vision towers of the Qwen3-Omni thinker, laid out like the Hugging Face checkpoint
(``thinker.audio_tower.*`` / ``thinker.visual.*``; the reference builds them from vLLM's and
transformers' modules: vllm_omni/model_executor/models/qwen3_omni/qwen3_omni_moe_thinker.py).

Audio: the mel spectrogram is cut into chunks of ``2 * n_window`` frames; every chunk goes
through three stride-2 3x3 convolutions (GELU), a linear layer over (channel, mel) and gets a
sinusoidal position that restarts per chunk; the valid frames of all chunks are then encoded by
pre-LN transformer layers whose attention is block-diagonal over windows of
``n_window_infer / (2 n_window)`` chunks, and projected to the thinker width.

Vision: linear patch embedding of (C, t, p, p) patches in merge-group order, a learned position
grid interpolated bilinearly to the image's patch grid, 2-D rotary attention inside each frame,
a 2x2 patch merger at the end and "deep-stack" mergers after selected blocks, whose outputs are
added to the first decoder layers' hidden states at the image positions.

Linear layers and norms run through the same sm_100a ops as the decoders (``FusedLinear``,
``norm_modulate``); q/k/v are stacked at load time.  The tcgen05 attention kernel covers head
size 128; these towers use 64 / 72-wide heads, so their (short-window) attention goes through
the fp32 formula.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from ...diffusion.layers.linear import FusedLinear
from ...ops import fused
from ...ops.attention import attention, attention_reference
from .config import AudioEncoderConfig, VisionEncoderConfig


def _mha(q, k, v, kv_lens=None):
    """[B, S, H, D] non-causal attention with an optional per-batch key length."""
    if q.is_cuda and q.shape[-1] in (64, 128) and q.dtype == torch.bfloat16:
        return attention(q, k, v, kv_lens=kv_lens)
    return attention_reference(q, k, v, kv_lens=kv_lens)


def _act(x, name):
    if name in ("gelu_pytorch_tanh", "gelu_tanh"):
        return F.gelu(x.float(), approximate="tanh").to(x.dtype)
    if name == "silu":
        return F.silu(x)
    return F.gelu(x.float()).to(x.dtype)


class EncoderBlock(nn.Module):
    """Pre-LN block: LayerNorm, MHA (stacked qkv with bias), LayerNorm, two-layer MLP."""

    def __init__(self, dim, heads, ffn, eps, act, dtype, device):
        super().__init__()
        self.heads, self.eps, self.act = heads, eps, act
        P = lambda v: nn.Parameter(torch.full((dim,), v, dtype=dtype, device=device), requires_grad=False)
        self.ln1_w, self.ln1_b, self.ln2_w, self.ln2_b = P(1.0), P(0.0), P(1.0), P(0.0)
        self.qkv = FusedLinear(dim, 3 * dim, dtype=dtype, device=device)
        self.proj = FusedLinear(dim, dim, dtype=dtype, device=device)
        self.fc1 = FusedLinear(dim, ffn, dtype=dtype, device=device)
        self.fc2 = FusedLinear(ffn, dim, dtype=dtype, device=device)

    def forward(self, x, kv_lens=None, cos=None, sin=None):           # x: [B, S, D]
        B, S, D = x.shape
        H, Dh = self.heads, D // self.heads
        h = fused.norm_modulate(x, weight=self.ln1_w, bias=self.ln1_b, eps=self.eps)
        qkv = self.qkv(h)
        if cos is not None:
            if qkv.is_cuda and Dh not in (64, 128):
                qkv = fused.qk_norm_rope_reference(qkv, H, H, Dh, None, None, None, None, 1 << 30, cos, sin, False, self.eps)
            else:
                fused.qk_norm_rope_(qkv, H, H, Dh, cos=cos, sin=sin, interleaved=False, eps=self.eps)
        q5 = qkv.view(B, S, 3, H, Dh)
        o = _mha(q5[:, :, 0], q5[:, :, 1], q5[:, :, 2], kv_lens).reshape(B, S, D)
        x = self.proj(o.contiguous(), residual=x)
        h = fused.norm_modulate(x, weight=self.ln2_w, bias=self.ln2_b, eps=self.eps)
        if self.act in ("gelu_pytorch_tanh", "gelu_tanh"):
            return self.fc2(self.fc1(h, act="gelu_tanh"), residual=x)
        return self.fc2(_act(self.fc1(h), self.act), residual=x)

    def load(self, rest: str, w, names: dict) -> bool:
        """``names``: checkpoint sub-name -> (attribute, slot) for this tower's naming."""
        if rest not in names:
            return False
        attr, slot = names[rest]
        D = self.ln1_w.shape[0]
        tgt = getattr(self, attr[0]) if len(attr) == 1 else getattr(getattr(self, attr[0]), attr[1])
        dst = tgt if slot is None else tgt[slot * D:(slot + 1) * D]
        dst.copy_(w.to(dst.dtype).reshape(dst.shape))
        return True


def _block_names(q, k, v, o, ln1, ln2, fc1, fc2, stacked_qkv=False):
    n = {}
    for suf in ("weight", "bias"):
        if stacked_qkv:
            n[f"{q}.{suf}"] = (("qkv", suf), None)
        else:
            n[f"{q}.{suf}"], n[f"{k}.{suf}"], n[f"{v}.{suf}"] = (("qkv", suf), 0), (("qkv", suf), 1), (("qkv", suf), 2)
        n[f"{o}.{suf}"] = (("proj", suf), None)
        n[f"{fc1}.{suf}"], n[f"{fc2}.{suf}"] = (("fc1", suf), None), (("fc2", suf), None)
    n[f"{ln1}.weight"], n[f"{ln1}.bias"] = (("ln1_w",), None), (("ln1_b",), None)
    n[f"{ln2}.weight"], n[f"{ln2}.bias"] = (("ln2_w",), None), (("ln2_b",), None)
    return n


_AUDIO_BLOCK = _block_names("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.out_proj",
                            "self_attn_layer_norm", "final_layer_norm", "fc1", "fc2")
_VISION_BLOCK = _block_names("attn.qkv", None, None, "attn.proj", "norm1", "norm2", "mlp.linear_fc1", "mlp.linear_fc2",
                             stacked_qkv=True)


def _halve3(n: int) -> int:
    for _ in range(3):
        n = (n - 1) // 2 + 1
    return n


class AudioEncoder(nn.Module):
    """mel [n_mels, T] -> [N, output_dim], N = sum over chunks of the thrice-halved chunk length."""

    def __init__(self, cfg: AudioEncoderConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        c = cfg.downsample_hidden_size
        kw = dict(dtype=dtype, device=device)
        self.conv2d1 = nn.Conv2d(1, c, 3, 2, 1, **kw)
        self.conv2d2 = nn.Conv2d(c, c, 3, 2, 1, **kw)
        self.conv2d3 = nn.Conv2d(c, c, 3, 2, 1, **kw)
        self.conv_out = FusedLinear(c * _halve3(cfg.num_mel_bins), cfg.d_model, bias=False, **kw)
        self.layers = nn.ModuleList([EncoderBlock(cfg.d_model, cfg.encoder_attention_heads, cfg.encoder_ffn_dim, 1e-5,
                                                  cfg.activation_function, dtype, device)
                                     for _ in range(cfg.encoder_layers)])
        self.ln_post_w = nn.Parameter(torch.ones(cfg.d_model, **kw), requires_grad=False)
        self.ln_post_b = nn.Parameter(torch.zeros(cfg.d_model, **kw), requires_grad=False)
        self.proj1 = FusedLinear(cfg.d_model, cfg.d_model, **kw)
        self.proj2 = FusedLinear(cfg.d_model, cfg.output_dim, **kw)

    def output_length(self, n_frames: int) -> int:
        W = 2 * self.cfg.n_window
        full, tail = divmod(n_frames, W)
        return full * _halve3(W) + (_halve3(tail) if tail else 0)

    @torch.no_grad()
    def forward(self, mel: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        W = 2 * cfg.n_window
        n_mels, T = mel.shape
        n_chunks = max(1, -(-T // W))
        x = mel.to(self.conv2d1.weight.dtype)
        if n_chunks == 1:
            x = x[None, None]                                                 # a single chunk keeps its own length
        else:
            if n_chunks * W != T:
                x = F.pad(x, (0, n_chunks * W - T))                           # short last chunk: zero frames
            x = x.view(n_mels, n_chunks, W).permute(1, 0, 2)[:, None]         # [chunks, 1, n_mels, W]
        x = F.gelu(self.conv2d1(x))
        x = F.gelu(self.conv2d2(x))
        x = F.gelu(self.conv2d3(x))                                          # [chunks, C, F', t]
        nc, C, Fq, t = x.shape
        x = self.conv_out(x.permute(0, 3, 1, 2).reshape(nc, t, C * Fq).contiguous())
        x = x + self._sinusoid(t, x.shape[-1], x.device).to(x.dtype)[None]
        tail = T - (n_chunks - 1) * W
        valid = [t] * (n_chunks - 1) + [_halve3(tail)]
        x = torch.cat([x[i, :n] for i, n in enumerate(valid)]) if valid[-1] != t else x.reshape(nc * t, -1)
        N, D = x.shape
        # block-diagonal attention: windows become the batch, the last one is shorter
        win = _halve3(W) * max(1, cfg.n_window_infer // W)
        n_win = -(-N // win)
        xb = F.pad(x, (0, 0, 0, n_win * win - N)).view(n_win, win, D).contiguous()
        lens = torch.full((n_win,), win, dtype=torch.int32, device=x.device)
        lens[-1] = N - (n_win - 1) * win
        kv_lens = lens if int(lens[-1]) != win else None
        for blk in self.layers:
            xb = blk(xb, kv_lens)
        x = xb.view(n_win * win, D)[:N].contiguous()
        x = fused.norm_modulate(x, weight=self.ln_post_w, bias=self.ln_post_b, eps=1e-5)
        return self.proj2(_act(self.proj1(x), cfg.activation_function))

    @staticmethod
    def _sinusoid(n, dim, device):
        half = dim // 2
        inv = torch.exp(-math.log(10000.0) / max(half - 1, 1) * torch.arange(half, device=device).float())
        ang = torch.arange(n, device=device).float()[:, None] * inv[None]
        return torch.cat([ang.sin(), ang.cos()], dim=-1)

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        """Names relative to ``thinker.audio_tower.``."""
        simple = {"conv2d1.weight": self.conv2d1.weight, "conv2d1.bias": self.conv2d1.bias,
                  "conv2d2.weight": self.conv2d2.weight, "conv2d2.bias": self.conv2d2.bias,
                  "conv2d3.weight": self.conv2d3.weight, "conv2d3.bias": self.conv2d3.bias,
                  "conv_out.weight": self.conv_out.weight, "ln_post.weight": self.ln_post_w, "ln_post.bias": self.ln_post_b,
                  "proj1.weight": self.proj1.weight, "proj1.bias": self.proj1.bias,
                  "proj2.weight": self.proj2.weight, "proj2.bias": self.proj2.bias}
        loaded = set()
        for n, w in weights:
            if n in simple:
                simple[n].copy_(w.to(simple[n].dtype))
                loaded.add(n)
            elif n.startswith("layers."):
                p = n.split(".")
                if self.layers[int(p[1])].load(".".join(p[2:]), w, _AUDIO_BLOCK):
                    loaded.add(n)
        return loaded


class PatchMerger(nn.Module):
    """LayerNorm (before or after grouping m x m neighbours), Linear, GELU, Linear."""

    def __init__(self, cfg: VisionEncoderConfig, post_shuffle_norm: bool, dtype, device):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.group = cfg.hidden_size * cfg.spatial_merge_size ** 2
        self.post = post_shuffle_norm
        n = self.group if post_shuffle_norm else cfg.hidden_size
        self.ln_w = nn.Parameter(torch.ones(n, **kw), requires_grad=False)
        self.ln_b = nn.Parameter(torch.zeros(n, **kw), requires_grad=False)
        self.fc1 = FusedLinear(self.group, self.group, **kw)
        self.fc2 = FusedLinear(self.group, cfg.out_hidden_size, **kw)

    def forward(self, x):           # [N, hidden]
        x = x.reshape(-1, self.group) if self.post else x
        x = fused.norm_modulate(x.contiguous(), weight=self.ln_w, bias=self.ln_b, eps=1e-6).reshape(-1, self.group)
        return self.fc2(F.gelu(self.fc1(x.contiguous()).float()).to(x.dtype))

    def load(self, rest, w) -> bool:
        tgt = {"ln_q.weight": self.ln_w, "ln_q.bias": self.ln_b, "mlp.0.weight": self.fc1.weight, "mlp.0.bias": self.fc1.bias,
               "mlp.2.weight": self.fc2.weight, "mlp.2.bias": self.fc2.bias}.get(rest)
        if tgt is None:
            return False
        tgt.copy_(w.to(tgt.dtype))
        return True


class VisionEncoder(nn.Module):
    """pixels [T, C, H, W] -> (merged embeddings [T' (H/p/m) (W/p/m), out_hidden], merged grid,
    deep-stack features: one tensor of the same shape per entry of ``deepstack_visual_indexes``)."""

    def __init__(self, cfg: VisionEncoderConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        kw = dict(dtype=dtype, device=device)
        pd = cfg.in_channels * cfg.temporal_patch_size * cfg.patch_size * cfg.patch_size
        self.patch_embed = FusedLinear(pd, cfg.hidden_size, **kw)
        self.pos_embed = nn.Parameter(torch.empty(cfg.num_position_embeddings, cfg.hidden_size, **kw).normal_(0, 0.02),
                                      requires_grad=False)
        self.blocks = nn.ModuleList([EncoderBlock(cfg.hidden_size, cfg.num_heads, cfg.intermediate_size, 1e-6,
                                                  cfg.hidden_act, dtype, device) for _ in range(cfg.depth)])
        self.merger = PatchMerger(cfg, False, dtype, device)
        self.deepstack = tuple(i for i in cfg.deepstack_visual_indexes if i < cfg.depth)
        self.merger_list = nn.ModuleList([PatchMerger(cfg, True, dtype, device) for _ in self.deepstack])
        Dh = cfg.hidden_size // cfg.num_heads
        self.inv_freq = 1.0 / (10000.0 ** (torch.arange(0, Dh // 2, 2, dtype=torch.float32) / (Dh // 2)))

    def grid(self, T, H, W):
        c = self.cfg
        return max(1, T // c.temporal_patch_size), H // c.patch_size, W // c.patch_size

    def _merge_order(self, t, gh, gw):
        """Patch (y, x) coordinates in the order of the token sequence: m x m groups contiguous."""
        m = self.cfg.spatial_merge_size
        ys = torch.arange(gh).view(gh // m, 1, m, 1).expand(gh // m, gw // m, m, m).reshape(-1)
        xs = torch.arange(gw).view(1, gw // m, 1, m).expand(gh // m, gw // m, m, m).reshape(-1)
        return ys, xs

    def _pos_embed(self, gh, gw, device):
        """Learned G x G position grid sampled bilinearly at gh x gw points, in token order."""
        G = int(self.cfg.num_position_embeddings ** 0.5)
        hy, wx = torch.linspace(0, G - 1, gh), torch.linspace(0, G - 1, gw)
        y0, x0 = hy.int(), wx.int()
        y1, x1 = (y0 + 1).clamp(max=G - 1), (x0 + 1).clamp(max=G - 1)
        dy, dx = (hy - y0)[:, None], (wx - x0)[None, :]
        pe = self.pos_embed.float()
        at = lambda yy, xx: pe[(yy[:, None] * G + xx[None, :]).long().to(device)]          # [gh, gw, D]
        w = lambda a: a.to(device)[..., None]
        grid = at(y0, x0) * w((1 - dy) * (1 - dx)) + at(y0, x1) * w((1 - dy) * dx) + \
            at(y1, x0) * w(dy * (1 - dx)) + at(y1, x1) * w(dy * dx)
        ys, xs = self._merge_order(1, gh, gw)
        return grid[ys.to(device), xs.to(device)]                                          # [gh*gw, D]

    def _rope(self, gh, gw, device):
        ys, xs = self._merge_order(1, gh, gw)
        inv = self.inv_freq.to(device)
        ang = torch.cat([ys.to(device).float()[:, None] * inv[None], xs.to(device).float()[:, None] * inv[None]], dim=-1)
        return ang.cos().contiguous(), ang.sin().contiguous()                              # [gh*gw, Dh/2]

    @torch.no_grad()
    def forward(self, pixels: torch.Tensor):
        c = self.cfg
        T, C, H, W = pixels.shape
        if T % c.temporal_patch_size:
            pixels = torch.cat([pixels, pixels[-1:].expand(c.temporal_patch_size - T % c.temporal_patch_size, -1, -1, -1)])
            T = pixels.shape[0]
        gt, gh, gw = self.grid(T, H, W)
        p, m = c.patch_size, c.spatial_merge_size
        x = pixels[:, :, :gh * p, :gw * p].reshape(gt, c.temporal_patch_size, C, gh // m, m, p, gw // m, m, p)
        # (frame, block row, block col, row in block, col in block) x (C, t, p, p)
        x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8).reshape(gt * gh * gw, -1)
        return self.forward_patches(x, (gt, gh, gw))

    @torch.no_grad()
    def forward_patches(self, patches: torch.Tensor, grid_thw):
        """patches: [t*h*w, C*tp*p*p] already in merge-group order (the HF image processor's layout)."""
        c = self.cfg
        gt, gh, gw = grid_thw
        m = c.spatial_merge_size
        dev = patches.device
        x = self.patch_embed(patches.to(self.pos_embed.dtype).contiguous())
        x = (x.view(gt, gh * gw, -1) + self._pos_embed(gh, gw, dev).to(x.dtype)[None]).contiguous()
        cos, sin = self._rope(gh, gw, dev)
        deep = []
        for i, blk in enumerate(self.blocks):
            x = blk(x, None, cos, sin)                                       # attention inside each frame
            if i in self.deepstack:
                deep.append(self.merger_list[self.deepstack.index(i)](x.reshape(gt * gh * gw, -1)))
        out = self.merger(x.reshape(gt * gh * gw, -1))
        return out, (gt, gh // m, gw // m), deep

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        """Names relative to ``thinker.visual.``."""
        loaded = set()
        for n, w in weights:
            p = n.split(".")
            ok = False
            if n == "patch_embed.proj.weight":
                self.patch_embed.weight.copy_(w.to(self.patch_embed.weight.dtype).reshape(self.patch_embed.weight.shape))
                ok = True
            elif n == "patch_embed.proj.bias":
                self.patch_embed.bias.copy_(w.to(self.patch_embed.bias.dtype))
                ok = True
            elif n == "pos_embed.weight":
                self.pos_embed.copy_(w.to(self.pos_embed.dtype))
                ok = True
            elif p[0] == "blocks":
                ok = self.blocks[int(p[1])].load(".".join(p[2:]), w, _VISION_BLOCK)
            elif p[0] == "merger":
                ok = self.merger.load(".".join(p[1:]), w)
            elif p[0] == "merger_list" and int(p[1]) < len(self.merger_list):
                ok = self.merger_list[int(p[1])].load(".".join(p[2:]), w)
            if ok:
                loaded.add(n)
        return loaded
