"""Qwen3-Omni code2wav stage: codec frames [T, G] -> 24 kHz waveform.

Mean of the per-codebook embeddings (one table, codebook g at offset g * codebook_size) ->
sliding-window causal transformer with RoPE and layer scale -> (transposed conv, ConvNeXt block)
per ``upsampling_ratios`` -> causal conv -> one block per ``upsample_rates`` (SnakeBeta, transposed
conv, three dilated residual units) -> SnakeBeta -> causal conv to one channel, clamped to
[-1, 1].  Long sequences are decoded in chunks of ``chunk_size`` frames with ``left_context``
frames of overlap whose samples are discarded
(vllm_omni/model_executor/models/qwen3_omni/qwen3_omni_code2wav.py:35-255).  The module tree
and parameter names follow the Hugging Face checkpoint (``code2wav.*``), except that q/k/v and
gate/up are stacked at load time.  A one-shot ("generation") stage: no sampling, no KV cache.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from ...diffusion.layers.linear import FusedLinear
from ...ops import conv as CV
from ...ops import fused
from ..base import StageModel
from .config import Code2WavConfig, Qwen3OmniConfig


def use_channels_last(model, x) -> bool:
    """GPU bf16 runs take the channels-last vocoder kernels (``OMNI_VOCODER_NLC=0`` keeps the library
    convolutions); ``model.vocoder_layout`` = "nlc" / "nct" forces either (tests)."""
    forced = getattr(model, "vocoder_layout", None)
    if forced is not None:
        return forced == "nlc"
    import os
    return x.is_cuda and x.dtype == torch.bfloat16 and os.environ.get("OMNI_VOCODER_NLC", "1") != "0"


class SnakeBeta(nn.Module):
    """x + sin^2(x e^alpha) / e^beta, per channel."""

    def __init__(self, ch, dtype, device):
        super().__init__()
        self.alpha = nn.Parameter(torch.zeros(ch, dtype=dtype, device=device), requires_grad=False)
        self.beta = nn.Parameter(torch.zeros(ch, dtype=dtype, device=device), requires_grad=False)

    def forward(self, x):           # x: [B, C, T]
        a = self.alpha.float().exp()[None, :, None]
        b = self.beta.float().exp()[None, :, None]
        xf = x.float()
        return (xf + (1.0 / (b + 1e-9)) * torch.sin(xf * a).pow(2)).to(x.dtype)

    def forward_nlc(self, x):       # x: [B, T, C]; one fused kernel on the GPU
        key = (self.alpha._version, self.beta._version)
        if getattr(self, "_ab", None) is None or self._ab[0] != key:
            self._ab = (key, self.alpha.float().exp().contiguous(), (1.0 / (self.beta.float().exp() + 1e-9)).contiguous())
        return CV.snake_nlc(x, self._ab[1], self._ab[2])


class CausalConv1d(nn.Module):
    """Left-padded convolution: output t sees inputs <= t (parameters ``conv.weight/bias``)."""

    def __init__(self, cin, cout, k, dilation=1, stride=1, groups=1, dtype=None, device=None):
        super().__init__()
        self.conv = nn.Conv1d(cin, cout, k, stride=stride, dilation=dilation, groups=groups, dtype=dtype, device=device)
        self.k_eff, self.stride = (k - 1) * dilation + 1, stride
        self.pad = self.k_eff - stride

    def forward(self, x):
        L = x.shape[-1]
        frames = math.ceil((L - self.k_eff + self.pad) / self.stride + 1)
        extra = (frames - 1) * self.stride + (self.k_eff - self.pad) - L
        return self.conv(F.pad(x, (self.pad, extra)))

    def forward_nlc(self, x, residual=None):
        """Channels-last twin ([B, T, C] in and out, stride 1): the implicit-GEMM convolution of ops/conv.py,
        or the depthwise kernel when every channel is its own group."""
        cv = self.conv
        assert self.stride == 1
        k, dil = cv.kernel_size[0], cv.dilation[0]
        key = (cv.weight._version, x.dtype)
        if getattr(self, "_pk", None) is None or self._pk[0] != key:
            if cv.groups == 1:
                self._pk = (key,) + CV.pack_conv1d_weight(cv.weight.data, cv.bias.data if cv.bias is not None else None, x.dtype)
            else:
                assert cv.groups == cv.in_channels == cv.out_channels
                self._pk = (key, cv.weight.data[:, 0].t().float().contiguous(),
                            cv.bias.data.float().contiguous() if cv.bias is not None else None)
        if cv.groups != 1:
            y = CV.dwconv1d_nlc(x.contiguous(), self._pk[1], self._pk[2], k, dil, self.pad)
            return y if residual is None else y + residual
        y = CV.conv1d_nlc(x, self._pk[1], self._pk[2], k, cv.in_channels, dil, self.pad, residual=residual)
        return y if y.shape[-1] == cv.out_channels else y[..., :cv.out_channels]


class CausalTransConv1d(nn.Module):
    """Transposed convolution with (kernel - stride) samples cut from both ends (Qwen3-Omni code2wav)
    or, with ``trim_left=False``, from the right end only (the Qwen3-TTS 12 Hz tokenizer decoder)."""

    def __init__(self, cin, cout, k, stride, dtype=None, device=None, trim_left=True):
        super().__init__()
        self.conv = nn.ConvTranspose1d(cin, cout, k, stride=stride, dtype=dtype, device=device)
        self.trim = k - stride
        self.left = self.trim if trim_left else 0

    def forward(self, x):
        y = self.conv(x)
        return y[..., self.left: y.shape[-1] - self.trim].contiguous()

    def forward_nlc(self, x):
        """[B, T, Cin] -> [B, T_out, Cout]: all output phases from one stride-1 convolution on weights
        stacked by phase (ops/conv.pack_conv_transpose1d_weight)."""
        cv = self.conv
        k, r = cv.kernel_size[0], cv.stride[0]
        key = (cv.weight._version, x.dtype)
        if getattr(self, "_pk", None) is None or self._pk[0] != key:
            self._pk = (key, CV.pack_conv_transpose1d_weight(cv.weight.data, cv.bias.data if cv.bias is not None else None,
                                                             r, self.left, x.dtype))
        t_out = (x.shape[1] - 1) * r + k - self.left - self.trim
        y = CV.conv_transpose1d_nlc(x, self._pk[1], cv.in_channels, r, t_out)
        return y if y.shape[-1] == cv.out_channels else y[..., :cv.out_channels]


class ConvNeXtBlock(nn.Module):
    def __init__(self, dim, dtype, device):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.dwconv = CausalConv1d(dim, dim, 7, groups=dim, **kw)
        self.norm = nn.LayerNorm(dim, eps=1e-6, **kw)
        self.pwconv1 = FusedLinear(dim, 4 * dim, **kw)
        self.pwconv2 = FusedLinear(4 * dim, dim, **kw)
        self.gamma = nn.Parameter(torch.full((dim,), 1e-6, **kw), requires_grad=False)

    def forward(self, x):           # [B, C, T]
        h = self.norm(self.dwconv(x).transpose(1, 2))
        h = self.pwconv2(F.gelu(self.pwconv1(h.contiguous())))
        return x + (self.gamma * h).transpose(1, 2)

    def forward_nlc(self, x):       # [B, T, C]
        h = F.layer_norm(self.dwconv.forward_nlc(x), (x.shape[-1],), self.norm.weight, self.norm.bias, self.norm.eps)
        h = F.gelu(self.pwconv1(h))
        return self.pwconv2(h, gate=self.gamma.view(1, -1), residual=x)      # x + gamma * pwconv2(h) in the GEMM epilogue


class ResUnit(nn.Module):
    def __init__(self, ch, dilation, dtype, device):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.act1, self.act2 = SnakeBeta(ch, dtype, device), SnakeBeta(ch, dtype, device)
        self.conv1 = CausalConv1d(ch, ch, 7, dilation=dilation, **kw)
        self.conv2 = CausalConv1d(ch, ch, 1, **kw)

    def forward(self, x):
        return x + self.conv2(self.act2(self.conv1(self.act1(x))))

    def forward_nlc(self, x):
        h = self.conv1.forward_nlc(self.act1.forward_nlc(x))
        return self.conv2.forward_nlc(self.act2.forward_nlc(h), residual=x)   # the skip rides in the epilogue


class DecoderBlock(nn.Module):
    """``block.0`` SnakeBeta, ``block.1`` transposed conv (x rate), ``block.2-4`` residual units."""

    def __init__(self, cin, cout, rate, dtype, device, trim_left=True):
        super().__init__()
        self.block = nn.ModuleList([SnakeBeta(cin, dtype, device),
                                    CausalTransConv1d(cin, cout, 2 * rate, rate, dtype=dtype, device=device,
                                                      trim_left=trim_left)] +
                                   [ResUnit(cout, d, dtype, device) for d in (1, 3, 9)])

    def forward(self, x):
        for b in self.block:
            x = b(x)
        return x

    def forward_nlc(self, x):
        for b in self.block:
            x = b.forward_nlc(x)
        return x


class WindowLayer(nn.Module):
    """Pre-norm transformer layer: causal attention inside a sliding window, RoPE, SwiGLU MLP, both
    residual branches scaled per channel (layer scale)."""

    def __init__(self, cfg: Code2WavConfig, dtype, device):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        D, H, Hkv = cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads
        self.H, self.Hkv, self.Dh, self.window, self.eps = H, Hkv, cfg.head_dim or D // H, cfg.sliding_window, cfg.rms_norm_eps
        P = lambda v: nn.Parameter(torch.full((D,), v, **kw), requires_grad=False)
        self.input_layernorm, self.post_attention_layernorm = P(1.0), P(1.0)
        self.attn_scale, self.mlp_scale = P(cfg.layer_scale_initial_scale), P(cfg.layer_scale_initial_scale)
        self.qkv = FusedLinear(D, (H + 2 * Hkv) * self.Dh, bias=cfg.attention_bias, **kw)
        self.o = FusedLinear(H * self.Dh, D, bias=cfg.attention_bias, **kw)
        self.gate_up = FusedLinear(D, 2 * cfg.intermediate_size, bias=False, **kw)
        self.down = FusedLinear(cfg.intermediate_size, D, bias=False, **kw)

    def forward(self, x, cos, sin, mask):           # x [B, T, D]
        B, T, D = x.shape
        H, Hkv, Dh = self.H, self.Hkv, self.Dh
        h = fused.norm_modulate(x, weight=self.input_layernorm, rms=True, eps=self.eps)
        qkv = self.qkv(h)
        if qkv.is_cuda and Dh not in (64, 128):
            qkv = fused.qk_norm_rope_reference(qkv, H, Hkv, Dh, None, None, None, None, 1 << 30, cos, sin, False, self.eps)
        else:
            fused.qk_norm_rope_(qkv, H, Hkv, Dh, cos=cos, sin=sin, interleaved=False, eps=self.eps)
        q = qkv[..., :H * Dh].view(B, T, H, Dh).transpose(1, 2)
        k = qkv[..., H * Dh:(H + Hkv) * Dh].view(B, T, Hkv, Dh).transpose(1, 2)
        v = qkv[..., (H + Hkv) * Dh:].view(B, T, Hkv, Dh).transpose(1, 2)
        if Hkv != H:
            k, v = k.repeat_interleave(H // Hkv, dim=1), v.repeat_interleave(H // Hkv, dim=1)
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=mask).transpose(1, 2).reshape(B, T, H * Dh)
        x = x + self.attn_scale * self.o(o.contiguous())
        h = fused.norm_modulate(x.contiguous(), weight=self.post_attention_layernorm, rms=True, eps=self.eps)
        return x + self.mlp_scale * self.down(fused.silu_mul(self.gate_up(h)))


class PreTransformer(nn.Module):
    def __init__(self, cfg: Code2WavConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        self.layers = nn.ModuleList([WindowLayer(cfg, dtype, device) for _ in range(cfg.num_hidden_layers)])
        self.norm = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype, device=device), requires_grad=False)
        Dh = cfg.head_dim or cfg.hidden_size // cfg.num_attention_heads
        self.inv_freq = 1.0 / (cfg.rope_theta ** (torch.arange(0, Dh, 2, dtype=torch.float32) / Dh))

    def forward(self, x):
        T = x.shape[1]
        i = torch.arange(T, device=x.device)
        ang = i.float()[:, None] * self.inv_freq.to(x.device)[None]
        cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
        mask = (i[None, :] <= i[:, None]) & (i[:, None] - i[None, :] < self.cfg.sliding_window)
        for layer in self.layers:
            x = layer(x, cos, sin, mask)
        return fused.norm_modulate(x.contiguous(), weight=self.norm, rms=True, eps=self.cfg.rms_norm_eps)


def pre_transformer_target(pt: "PreTransformer", n: str):
    """Checkpoint name ``pre_transformer.*`` -> (parameter, row slice or None) of the fused layout."""
    c = pt.cfg
    p = n.split(".")
    if n == "pre_transformer.norm.weight":
        return pt.norm, None
    if not n.startswith("pre_transformer.layers."):
        return None, None
    layer = pt.layers[int(p[2])]
    rest = ".".join(p[3:])
    H, Hkv, Dh, Fi = layer.H, layer.Hkv, layer.Dh, c.intermediate_size
    qo = {"q_proj": (0, H * Dh), "k_proj": (H * Dh, (H + Hkv) * Dh), "v_proj": ((H + Hkv) * Dh, (H + 2 * Hkv) * Dh)}
    if p[3] == "self_attn" and p[4] in qo:
        return getattr(layer.qkv, p[5]), qo[p[4]]
    if p[3] == "self_attn" and p[4] == "o_proj":
        return getattr(layer.o, p[5]), None
    if rest == "mlp.gate_proj.weight":
        return layer.gate_up.weight, (0, Fi)
    if rest == "mlp.up_proj.weight":
        return layer.gate_up.weight, (Fi, 2 * Fi)
    if rest == "mlp.down_proj.weight":
        return layer.down.weight, None
    return {"input_layernorm.weight": layer.input_layernorm,
            "post_attention_layernorm.weight": layer.post_attention_layernorm,
            "self_attn_layer_scale.scale": layer.attn_scale,
            "mlp_layer_scale.scale": layer.mlp_scale}.get(rest), None


class Qwen3OmniCode2Wav(StageModel):
    engine_output_type = "audio"
    is_generation_model = True

    def __init__(self, cfg: Qwen3OmniConfig, dtype=torch.bfloat16, device=None):
        super().__init__(None, dtype, device)
        c = self.c = cfg.code2wav
        kw = dict(dtype=dtype, device=device)
        D = c.hidden_size
        self.code_embedding = nn.Parameter(torch.empty(c.num_quantizers * c.codebook_size, D, **kw).normal_(0, 0.02),
                                           requires_grad=False)
        self.pre_transformer = PreTransformer(c, dtype, device)
        self.upsample = nn.ModuleList([nn.ModuleList([CausalTransConv1d(D, D, r, r, **kw), ConvNeXtBlock(D, dtype, device)])
                                       for r in c.upsampling_ratios])
        dec = [CausalConv1d(D, c.decoder_dim, 7, **kw)]
        for i, r in enumerate(c.upsample_rates):
            dec.append(DecoderBlock(c.decoder_dim // 2 ** i, c.decoder_dim // 2 ** (i + 1), r, dtype, device))
        out = c.decoder_dim // 2 ** len(c.upsample_rates)
        dec += [SnakeBeta(out, dtype, device), CausalConv1d(out, 1, 7, **kw)]
        self.decoder = nn.ModuleList(dec)

    @torch.no_grad()
    def decode(self, codes: torch.Tensor) -> torch.Tensor:
        """codes: [B, G, T] int64 -> waveform [B, ~T * total_upsample] in [-1, 1] (every transposed
        convolution of the decoder drops ``rate`` samples at each end)."""
        c = self.c
        B, G, T = codes.shape
        if G != c.num_quantizers:
            raise ValueError(f"expected {c.num_quantizers} codebooks per frame, got {G}")
        off = torch.arange(G, device=codes.device)[None, :, None] * c.codebook_size
        x = self.code_embedding[codes.clamp(0, c.codebook_size - 1) + off].float().mean(1).to(self.code_embedding.dtype)
        x = self.pre_transformer(x.contiguous())
        if self._use_nlc(x):
            # channels-last all the way: the transformer's [B, T, D] output is the layout the 1-D implicit
            # GEMM, the depthwise kernel and the fused snake kernel work on
            for up, nxt in self.upsample:
                x = nxt.forward_nlc(up.forward_nlc(x))
            for blk in self.decoder:
                x = blk.forward_nlc(x)
            return x[..., 0].float().clamp(-1.0, 1.0)
        x = x.transpose(1, 2)
        for up, nxt in self.upsample:
            x = nxt(up(x))
        for blk in self.decoder:
            x = blk(x)
        return x.float().clamp(-1.0, 1.0)[:, 0]

    def _use_nlc(self, x) -> bool:
        return use_channels_last(self, x)

    @torch.no_grad()
    def chunked_decode(self, codes: torch.Tensor, chunk_size=None, left_context=None) -> torch.Tensor:
        c = self.c
        chunk_size = chunk_size or c.chunk_size
        left = c.left_context if left_context is None else left_context
        T = codes.shape[-1]
        up = c.total_upsample
        if T == 0:
            return torch.zeros(codes.shape[0], 0, device=codes.device)
        outs, start = [], 0
        while start < T:
            end = min(T, start + chunk_size)
            ctx = min(left, start)
            wav = self.decode(codes[..., start - ctx:end])
            outs.append(wav[..., ctx * up:])
            start = end
        return torch.cat(outs, dim=-1)[..., :T * up]

    def generate_for(self, req, start, n):
        info = req.additional_information
        codes = info.get("codes")
        if codes is None:                       # token ids carry a flattened [T * G] code list
            G = self.c.num_quantizers
            ids = torch.tensor(req.prompt_token_ids[start:start + n], dtype=torch.long)
            codes = ids[: (ids.numel() // G) * G].view(-1, G)
        codes = torch.as_tensor(codes).long().to(self.code_embedding.device)
        if codes.dim() == 2:                    # [T, G] -> [1, G, T]
            codes = codes.t()[None]
        ctx = int(info.get("left_context_frames", 0))
        wav = self.chunked_decode(codes)
        if ctx:
            wav = wav[..., ctx * self.c.total_upsample:]
        return {"audio": wav[0].float(), "sample_rate": self.c.sample_rate}

    # ------------------------------------------------------------------ weights
    @torch.no_grad()
    def load_weights(self, weights) -> set:
        """Checkpoint names under ``code2wav.``; other stages' tensors are ignored."""
        params = dict(self.named_parameters())
        loaded = set()
        for full, w in weights:
            if full.startswith(("thinker.", "talker.")):
                continue
            n = full[len("code2wav."):] if full.startswith("code2wav.") else full
            tgt, sl = None, None
            p = n.split(".")
            if n.startswith("pre_transformer."):
                tgt, sl = pre_transformer_target(self.pre_transformer, n)
            elif n == "code_embedding.weight":
                tgt = self.code_embedding
            else:
                tgt = params.get(n)
            if tgt is None:
                continue
            dst = tgt if sl is None else tgt[sl[0]:sl[1]]
            dst.copy_(w.to(dst.dtype).reshape(dst.shape))
            loaded.add(full)
        return loaded
