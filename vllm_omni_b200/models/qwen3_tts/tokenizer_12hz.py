"""Decoder of the Qwen3-TTS 12 Hz speech tokenizer: [B, G, T] codec frames -> 24 kHz waveform
(vllm_omni/model_executor/models/qwen3_tts/tokenizer_12hz/modeling_qwen3_tts_tokenizer_v2.py:662-879).

Front end: a split residual vector quantizer — codebook 0 (semantic) and codebooks 1..G-1
(acoustic) each sum their code vectors (``embedding_sum / cluster_usage``) in a space of half the
codebook width and map the sum through their own 1x1 convolution.  Because that map is linear it is
folded into the tables when the checkpoint is loaded: decoding a frame is ONE gather-and-sum over G
tables of the full codebook width.  Then a causal conv (k=3) to the latent width, a sliding-window
causal transformer between an input and an output projection, transposed-conv + ConvNeXt
upsampling stages and the SnakeBeta decoder blocks — the same blocks as Qwen3-Omni's code2wav,
except that its transposed convolutions cut their overhang from the right end only, so T frames
give exactly ``T * total_upsample`` samples.

Checkpoint names (under ``decoder.`` in the speech tokenizer's file): ``quantizer.rvq_first|rvq_rest.
vq.layers.N._codebook.{embedding_sum,cluster_usage}``, ``quantizer.rvq_*.output_proj.weight``,
``pre_conv.conv.*``, ``pre_transformer.{input_proj,output_proj,layers.N.*,norm}``, ``upsample.N.0|1.*``,
``decoder.N.*``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn

from ...diffusion.layers.linear import FusedLinear
from ..qwen3_omni.code2wav import (CausalConv1d, CausalTransConv1d, ConvNeXtBlock, DecoderBlock, PreTransformer, SnakeBeta,
                                   pre_transformer_target)
from ..qwen3_omni.config import Code2WavConfig


@dataclass
class TokenizerDecoderConfig(Code2WavConfig):
    codebook_dim: int = 512
    latent_dim: int = 1024

    @classmethod
    def from_dict(cls, d: dict) -> "TokenizerDecoderConfig":
        keys = set(cls.__dataclass_fields__)
        return cls(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in d.items() if k in keys})


class Qwen3TTSTokenizerDecoder(nn.Module):
    def __init__(self, cfg: TokenizerDecoderConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.c = c = cfg
        kw = dict(dtype=dtype, device=device)
        G, L = c.num_quantizers, c.latent_dim
        # folded quantizer tables: row g * codebook_size + code, already in the codebook_dim output space
        self.code_table = nn.Parameter(torch.empty(G * c.codebook_size, c.codebook_dim, **kw).normal_(0, 0.02),
                                       requires_grad=False)
        self.pre_conv = CausalConv1d(c.codebook_dim, L, 3, **kw)
        self.input_proj = FusedLinear(L, c.hidden_size, **kw)
        self.pre_transformer = PreTransformer(c, dtype, device)
        self.output_proj = FusedLinear(c.hidden_size, L, **kw)
        self.upsample = nn.ModuleList([nn.ModuleList([CausalTransConv1d(L, L, r, r, trim_left=False, **kw),
                                                      ConvNeXtBlock(L, dtype, device)]) for r in c.upsampling_ratios])
        dec = [CausalConv1d(L, c.decoder_dim, 7, **kw)]
        for i, r in enumerate(c.upsample_rates):
            dec.append(DecoderBlock(c.decoder_dim // 2 ** i, c.decoder_dim // 2 ** (i + 1), r, dtype, device, trim_left=False))
        out = c.decoder_dim // 2 ** len(c.upsample_rates)
        dec += [SnakeBeta(out, dtype, device), CausalConv1d(out, 1, 7, **kw)]
        self.decoder = nn.ModuleList(dec)

    @torch.no_grad()
    def decode(self, codes: torch.Tensor) -> torch.Tensor:
        """codes [B, G, T] int64 -> waveform [B, T * total_upsample] in [-1, 1]."""
        c = self.c
        B, G, T = codes.shape
        if G != c.num_quantizers:
            raise ValueError(f"expected {c.num_quantizers} codebooks per frame, got {G}")
        off = torch.arange(G, device=codes.device)[None, :, None] * c.codebook_size
        x = self.code_table[codes.clamp(0, c.codebook_size - 1) + off].float().sum(1).to(self.code_table.dtype)   # [B, T, cd]
        from ..qwen3_omni.code2wav import use_channels_last
        if use_channels_last(self, x):             # [B, T, C] throughout: own conv / snake kernels (ops/conv.py)
            x = self.pre_conv.forward_nlc(x.contiguous())
            x = self.output_proj(self.pre_transformer(self.input_proj(x.contiguous())))
            for up, nxt in self.upsample:
                x = nxt.forward_nlc(up.forward_nlc(x.contiguous()))
            for blk in self.decoder:
                x = blk.forward_nlc(x)
            return x[..., 0].float().clamp(-1.0, 1.0)
        x = self.pre_conv(x.transpose(1, 2)).transpose(1, 2).contiguous()
        x = self.output_proj(self.pre_transformer(self.input_proj(x))).transpose(1, 2)
        for up, nxt in self.upsample:
            x = nxt(up(x))
        for blk in self.decoder:
            x = blk(x)
        return x.float().clamp(-1.0, 1.0)[:, 0]

    @torch.no_grad()
    def chunked_decode(self, codes: torch.Tensor, chunk_size=None, left_context=None) -> torch.Tensor:
        """Decode in windows of ``chunk_size`` frames, each with ``left_context`` earlier frames whose
        samples are dropped (every layer is causal, so only the left side needs context)."""
        c = self.c
        chunk_size = chunk_size or c.chunk_size
        left = c.left_context if left_context is None else left_context
        T, up = codes.shape[-1], c.total_upsample
        if T == 0:
            return torch.zeros(codes.shape[0], 0, device=codes.device)
        outs, start = [], 0
        while start < T:
            end = min(T, start + chunk_size)
            ctx = left if start - left > 0 else start
            outs.append(self.decode(codes[..., start - ctx:end])[..., ctx * up:])
            start = end
        return torch.cat(outs, dim=-1)

    # ------------------------------------------------------------------ weights
    @torch.no_grad()
    def load_weights(self, weights) -> set:
        """Names relative to the tokenizer's ``decoder.`` module.  Quantizer pieces are collected and
        folded into ``code_table`` once all of them have been seen."""
        c = self.c
        params = dict(self.named_parameters())
        loaded, q = set(), {}
        for n, w in weights:
            tgt, sl = None, None
            if n.startswith("quantizer."):
                q[n] = w.float()
                continue
            if n.startswith("pre_transformer.input_proj."):
                tgt = getattr(self.input_proj, n.rsplit(".", 1)[1])
            elif n.startswith("pre_transformer.output_proj."):
                tgt = getattr(self.output_proj, n.rsplit(".", 1)[1])
            elif n.startswith("pre_transformer."):
                tgt, sl = pre_transformer_target(self.pre_transformer, n)
            else:
                tgt = params.get(n)
            if tgt is None:
                continue
            dst = tgt if sl is None else tgt[sl[0]:sl[1]]
            dst.copy_(w.to(dst.dtype).reshape(dst.shape))
            loaded.add(n)
        if q:
            table = self.code_table.view(c.num_quantizers, c.codebook_size, c.codebook_dim)
            for g in range(c.num_quantizers):
                grp, li = ("rvq_first", 0) if g == 0 else ("rvq_rest", g - 1)
                base = f"quantizer.{grp}.vq.layers.{li}._codebook."
                names = (base + "embedding_sum", base + "cluster_usage", f"quantizer.{grp}.output_proj.weight")
                if not all(k in q for k in names):
                    continue
                emb = q[names[0]] / q[names[1]].clamp(min=1e-5)[:, None]              # [bins, cd / 2]
                proj = q[names[2]].reshape(c.codebook_dim, -1)                        # conv1d 1x1 [cd, cd / 2, 1]
                table[g].copy_((emb @ proj.t()).to(table.dtype))
                loaded.update(names)
        return loaded
