"""Qwen3-Omni talker stage: a smaller MoE decoder that speaks codec frames.

Inputs (from the thinker, through ``thinker2talker``): the thinker's token embeddings and
layer-N hidden states for the whole sequence plus the tts bos/eos/pad embeddings.
Prefill: multimodal positions are projected with ``hidden_projection``, text positions with
``text_projection`` (vllm_omni/model_executor/models/qwen3_omni/qwen3_omni.py:586-917).
Decode: every step emits one codec frame of ``num_code_groups`` codes: code 0 is sampled from
the talker's codec head, codes 1..G-1 come from the code predictor, a small transformer run
G-1 times on (talker hidden, embeddings of the codes so far)
(qwen3_omni_moe_code_predictor_mtp.py:413-524).  The next input embedding is the sum of the
frame's code embeddings plus the projected thinker embedding of the next text token (or the
tts-pad embedding once the text is exhausted).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from ...diffusion.layers.linear import FusedLinear
from ...ops import fused
from ...ops.attention import attention_reference
from ...ops.sampler import RowParams, sample
from ..base import StageModel
from ..qwen_decoder import DecoderConfig, QwenDecoderModel
from .config import CodePredictorConfig, Qwen3OmniConfig


class ResizeMLP(nn.Module):
    """thinker width -> talker width: Linear, SiLU, Linear (checkpoint names ``linear_fc1/2``)."""

    def __init__(self, din, dhid, dout, dtype, device):
        super().__init__()
        self.fc1 = FusedLinear(din, dhid, dtype=dtype, device=device)
        self.fc2 = FusedLinear(dhid, dout, dtype=dtype, device=device)

    def forward(self, x):
        return self.fc2(self.fc1(x, act="silu"))

    def load_weights(self, weights) -> set:
        tgt = {"linear_fc1.weight": self.fc1.weight, "linear_fc1.bias": self.fc1.bias,
               "linear_fc2.weight": self.fc2.weight, "linear_fc2.bias": self.fc2.bias}
        loaded = set()
        for n, w in weights:
            if n in tgt:
                tgt[n].copy_(w.to(tgt[n].dtype))
                loaded.add(n)
        return loaded


class _PredictorState:
    """Static buffers of the cached code-predictor loop for one row-count bucket."""

    def __init__(self, n, core_cfg, talker_hidden, G, vocab, dtype, device):
        z = lambda *s, dt=dtype: torch.zeros(*s, dtype=dt, device=device)
        self.n = n
        page = 32                                    # one page per row holds the whole context (<= G + 1 tokens)
        self.page = page
        self.caches = [(z(n, page, core_cfg.num_key_value_heads, core_cfg.head_dim),
                        z(n, page, core_cfg.num_key_value_heads, core_cfg.head_dim))
                       for _ in range(core_cfg.num_hidden_layers)]
        self.tables = torch.arange(n, dtype=torch.int32, device=device)[:, None].contiguous()
        self.rows = torch.arange(n, dtype=torch.long, device=device)
        self.ids = torch.zeros(n, dtype=torch.long, device=device)
        self.emask = torch.ones(n, dtype=torch.bool, device=device)
        steps = G                                    # tokens fed: talker hidden, code 0, codes 1 .. G-2
        self.pos = [torch.full((n,), t, dtype=torch.long, device=device) for t in range(steps)]
        self.slots = [(torch.arange(n, dtype=torch.int32, device=device) * page + t).contiguous() for t in range(steps)]
        self.lens = [torch.full((n,), t + 1, dtype=torch.int32, device=device) for t in range(steps)]
        self.hidden_in, self.code0_in = z(n, talker_hidden), z(n, talker_hidden)
        self.codes = torch.zeros(n, G - 1, dtype=torch.long, device=device)
        self.summed = z(n, talker_hidden)
        self.sample_rows = None                      # uint8 [(G-1) * n * row_bytes] on the device when sampling
        self.sample_out = torch.zeros(n, dtype=torch.int32, device=device)
        self.sample_work = torch.zeros(n, vocab, dtype=torch.float32, device=device) if device.type == "cuda" else None
        self.graph, self.graph_mode, self.warm = None, None, 0


class CodePredictor(nn.Module):
    """G-1 sequential steps over a tiny context (<= G+1 tokens).  Every token is fed once: its K/V
    go to a one-page-per-row cache and attention is the paged decode kernel, and the whole loop
    (G decoder steps, G-1 heads, samplings and embedding look-ups) is captured in ONE CUDA graph per
    row-count bucket, because at these sizes it is launch-bound.  The reference runs it as CUDA
    graphs of a re-prefilled HF-style module (qwen3_omni_moe_code_predictor_mtp.py:413-524).
    ``generate_uncached`` is the straight restatement without a cache (the oracle of the tests)."""

    def __init__(self, cfg: CodePredictorConfig, talker_hidden: int, dtype, device):
        super().__init__()
        self.cfg = cfg
        dc = DecoderConfig(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
                           num_hidden_layers=cfg.num_hidden_layers, num_attention_heads=cfg.num_attention_heads,
                           num_key_value_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
                           intermediate_size=cfg.intermediate_size, rope_theta=cfg.rope_theta,
                           rms_norm_eps=cfg.rms_norm_eps)
        self.core = QwenDecoderModel(dc, dtype, device, with_lm_head=False)
        G = cfg.num_code_groups
        self.in_proj = FusedLinear(talker_hidden, cfg.hidden_size, dtype=dtype, device=device) \
            if talker_hidden != cfg.hidden_size else None
        # one embedding table and one head per residual codebook 1..G-1
        self.codec_embedding = nn.Parameter(torch.empty(G - 1, cfg.vocab_size, talker_hidden, dtype=dtype, device=device)
                                            .normal_(0, 0.02), requires_grad=False)
        self.lm_heads = nn.Parameter(torch.empty(G - 1, cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device)
                                     .normal_(0, 0.02), requires_grad=False)

    @torch.no_grad()
    def load_weights(self, weights) -> set:
        """Names relative to ``talker.code_predictor.``: ``model.layers.*`` / ``model.norm.weight``,
        ``model.codec_embedding.G.weight`` and ``lm_head.G.weight`` for residual codebooks G; Qwen3-TTS adds
        ``small_to_mtp_projection`` (talker width -> predictor width) when the two widths differ."""
        loaded, core = set(), []
        for n, w in weights:
            p = n.split(".")
            if n.startswith("model.codec_embedding.") and p[-1] == "weight":
                self.codec_embedding[int(p[2])].copy_(w.to(self.codec_embedding.dtype))
                loaded.add(n)
            elif n.startswith("lm_head.") and p[-1] == "weight":
                self.lm_heads[int(p[1])].copy_(w.to(self.lm_heads.dtype))
                loaded.add(n)
            elif n.startswith(("in_proj.", "small_to_mtp_projection.")) and self.in_proj is not None:
                getattr(self.in_proj, p[1]).copy_(w.to(self.in_proj.weight.dtype))
                loaded.add(n)
            else:
                core.append((n, w))
        return loaded | self.core.load_weights(core)

    def _forward_seq(self, x):
        """x: [n, L, D] small dense causal forward (no cache)."""
        from ..qwen_decoder import reference_forward  # noqa: F401  (same math, batched below)
        core, cfg = self.core, self.core.cfg
        n, L, D = x.shape
        H, Hkv, Dh = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        pos = torch.arange(L, device=x.device)
        cos, sin = core.rope.cos_sin_for(pos)
        x = x.reshape(n * L, D).contiguous()
        for layer in core.layers:
            xn = fused.norm_modulate(x, weight=layer.input_layernorm, rms=True, eps=cfg.rms_norm_eps)
            qkv = layer.qkv_proj(xn).view(n, L, -1)
            fused.qk_norm_rope_(qkv, H, Hkv, Dh, wq=layer.q_norm, wk=layer.k_norm, cos=cos, sin=sin,
                                interleaved=False, eps=cfg.rms_norm_eps)
            q = qkv[..., :H * Dh].reshape(n, L, H, Dh)
            k = qkv[..., H * Dh:(H + Hkv) * Dh].reshape(n, L, Hkv, Dh)
            v = qkv[..., (H + Hkv) * Dh:].reshape(n, L, Hkv, Dh)
            o = attention_reference(q, k, v, causal=True).reshape(n * L, H * Dh)
            layer.o_proj(o.contiguous(), residual=x, out=x)
            xn = fused.norm_modulate(x, weight=layer.post_attention_layernorm, rms=True, eps=cfg.rms_norm_eps)
            layer.down(fused.silu_mul(layer.gate_up(xn)), residual=x, out=x)
        return fused.norm_modulate(x, weight=core.norm, rms=True, eps=cfg.rms_norm_eps).view(n, L, D)

    # ------------------------------------------------------------------ cached loop
    def _bucket(self, n: int, device) -> "_PredictorState":
        nb = 1
        while nb < n:
            nb *= 2
        st = self._states.get((nb, str(device))) if hasattr(self, "_states") else None
        if st is None:
            if not hasattr(self, "_states"):
                self._states = {}
            st = _PredictorState(nb, self.core.cfg, self.codec_embedding.shape[-1], self.cfg.num_code_groups,
                                 self.cfg.vocab_size, self.codec_embedding.dtype, device)
            self._states[(nb, str(device))] = st
        return st

    def _loop_body(self, st: "_PredictorState", sampling: bool):
        """The whole frame on static buffers: reads st.hidden_in / st.code0_in (and st.sample_rows),
        writes st.codes / st.summed."""
        from ...ops.sampler import row_bytes, sample_packed
        from ..qwen_decoder import ModelBatch
        from ...ops import gemm
        G, n = self.cfg.num_code_groups, st.n
        st.summed.zero_()
        x = st.hidden_in
        for t in range(G):
            xin = x if self.in_proj is None else self.in_proj(x)
            b = ModelBatch(st.ids, st.pos[t], st.slots[t], [], decode_rows=st.rows, decode_block_tables=st.tables,
                           decode_seq_lens=st.lens[t], input_embeds=xin, embeds_mask=st.emask)
            h, _ = self.core(b, st.caches)                                    # [n, D]
            if t == 0:
                x = st.code0_in
                continue
            g = t - 1                                                          # this token predicts residual code g + 1
            if h.is_cuda:
                logits = gemm.linear(h, self.lm_heads[g])
            else:
                logits = F.linear(h.float(), self.lm_heads[g].float())
            if not sampling:
                c = logits.argmax(-1)
            elif h.is_cuda:
                rb = row_bytes() * n
                c = sample_packed(logits, st.sample_rows[g * rb:(g + 1) * rb], st.sample_out, st.sample_work).long()
            else:
                c = sample(logits, st.cpu_rows[g])[0].long()
            st.codes[:, g] = c
            e = self.codec_embedding[g][c]
            st.summed.add_(e)
            x = e

    @torch.no_grad()
    def generate(self, talker_hidden, code0_embed, temperature=0.0, seed=0, step=0):
        """talker_hidden, code0_embed: [n, Dt].  Returns (codes [n, G-1] int64, summed embeddings
        of codes 1..G-1 [n, Dt])."""
        import os
        from ...ops.sampler import pack_rows
        G, n, dev = self.cfg.num_code_groups, talker_hidden.shape[0], talker_hidden.device
        if G > 32 or self.core.cfg.head_dim not in (64, 128) and dev.type == "cuda":
            return self.generate_uncached(talker_hidden, code0_embed, temperature, seed, step)
        st = self._bucket(n, dev)
        st.hidden_in[:n].copy_(talker_hidden)
        st.code0_in[:n].copy_(code0_embed)
        if st.n > n:                                   # padding rows repeat row 0 (their results are dropped)
            st.hidden_in[n:].copy_(talker_hidden[:1].expand(st.n - n, -1))
            st.code0_in[n:].copy_(code0_embed[:1].expand(st.n - n, -1))
        sampling = temperature > 0
        if sampling:
            rows = [[RowParams(temperature=temperature, top_k=50, seed=seed + 7919 * (g + 1), step=step)
                     for _ in range(st.n)] for g in range(G - 1)]
            if dev.type == "cuda":
                packed = torch.cat([pack_rows(r) for r in rows]).to(dev, non_blocking=True)
                if st.sample_rows is None:
                    st.sample_rows = packed.clone()
                else:
                    st.sample_rows.copy_(packed)
            else:
                st.cpu_rows = rows
        use_graph = dev.type == "cuda" and os.environ.get("OMNI_PREDICTOR_GRAPH", "1") == "1"
        if not use_graph:
            self._loop_body(st, sampling)
        else:
            if st.graph is not None and st.graph_mode != sampling:
                st.graph, st.warm = None, 0            # greedy <-> sampling: capture again
            if st.graph is None:
                if st.warm < 1:
                    st.warm += 1
                    self._loop_body(st, sampling)      # eager once: builds workspaces, loads libraries
                else:
                    torch.cuda.synchronize()
                    g_ = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g_, capture_error_mode="thread_local"):   # other stages' threads keep issuing CUDA calls
                        self._loop_body(st, sampling)
                    st.graph, st.graph_mode = g_, sampling
                    st.graph.replay()
            else:
                st.graph.replay()
        return st.codes[:n].clone(), st.summed[:n].clone()

    @torch.no_grad()
    def generate_uncached(self, talker_hidden, code0_embed, temperature=0.0, seed=0, step=0):
        """Re-prefills the growing sequence at every step with plain fp32 attention: the oracle."""
        G = self.cfg.num_code_groups
        n = talker_hidden.shape[0]
        seq = torch.stack([talker_hidden, code0_embed], dim=1)               # [n, 2, Dt]
        codes, summed = [], torch.zeros_like(code0_embed)
        for g in range(G - 1):
            xin = seq if self.in_proj is None else self.in_proj(seq.contiguous())
            h = self._forward_seq(xin)[:, -1]                                # [n, D]
            logits = F.linear(h.float(), self.lm_heads[g].float())
            if temperature <= 0:
                c = logits.argmax(-1)
            else:
                c, _ = sample(logits, [RowParams(temperature=temperature, top_k=50, seed=seed + 7919 * (g + 1),
                                                 step=step) for _ in range(n)])
                c = c.long()
            e = self.codec_embedding[g][c]
            codes.append(c)
            summed = summed + e
            seq = torch.cat([seq, e[:, None]], dim=1)
        return torch.stack(codes, dim=1), summed


class Qwen3OmniMoeTalker(StageModel):
    engine_output_type = "latent"
    stream_output_keys = ("codes",)      # new codec frames ride on every streaming output

    def __init__(self, cfg: Qwen3OmniConfig, dtype=torch.bfloat16, device=None):
        super().__init__(cfg.talker, dtype, device)
        self.cfg = cfg
        Dt, Dth = cfg.talker.hidden_size, cfg.thinker.hidden_size
        self.decoder = QwenDecoderModel(cfg.talker, dtype, device, with_lm_head=False)
        Dr = cfg.talker.intermediate_size            # width of the resize MLPs' hidden layer
        self.text_projection = ResizeMLP(Dth, Dr, Dt, dtype, device)
        self.hidden_projection = ResizeMLP(Dth, Dr, Dt, dtype, device)
        self.codec_head = FusedLinear(Dt, cfg.talker.vocab_size, bias=False, dtype=dtype, device=device)
        self.code_predictor = CodePredictor(cfg.code_predictor, Dt, dtype, device)
        self.num_code_groups = cfg.code_predictor.num_code_groups

    def eos_token_id(self):
        return self.cfg.codec_eos_id

    # ---- request preprocessing (prefill embeddings)
    def speaker_token(self, voice: str | None) -> int:
        ids = self.cfg.speaker_ids
        if not ids:
            return self.cfg.audio_start_token_id
        return ids.get((voice or "").lower(), next(iter(ids.values())))

    @torch.no_grad()
    def preprocess_request(self, req) -> None:
        """Builds the talker prompt from the thinker's ChatML sequence
        (vllm_omni/model_executor/models/qwen3_omni/qwen3_omni.py:778-1005).  The sequence is cut at
        every ``<|im_start|>`` of the thinker prompt; system turns and earlier assistant turns are
        dropped; user turns contribute one row per token (multimodal rows: projected layer-N hidden
        state, text rows: projected embedding); the last assistant turn becomes nine rows,

            text side   h0 h1 h2 pad pad pad pad bos t0      (h = header tokens, t0 = first reply token)
            codec side   0  0  0 nothink think_bos think_eos speaker codec_pad codec_bos

        added row by row.  The remaining reply tokens followed by tts-eos are fed one per decode
        step on top of the previous frame's code embeddings, tts-pad afterwards.

        With ``thinker_stream`` in the request the thinker is still generating: the reply rows known so
        far are used, later ones arrive through ``on_stream_update``, and a decode step whose reply row
        has not arrived yet waits for it (``decode_blocked``) instead of guessing, so the frames equal
        those of the whole-request hand-off."""
        info = req.additional_information
        cfg = self.cfg
        dev = self.decoder.embed_tokens.device
        if "thinker_embeddings" not in info:
            return
        emb = info["thinker_embeddings"].to(dev, self.dtype_)               # [L_total, Dth]
        hid = info["thinker_hidden_states"].to(dev, self.dtype_)
        prompt_ids = list(info.get("thinker_input_ids") or [])
        seq = list(info.get("thinker_sequences") or prompt_ids)
        L = min(emb.shape[0], max(len(seq), len(prompt_ids)))
        n_in = min(len(prompt_ids), L)
        mm_ids = {cfg.audio_token_id, cfg.image_token_id, cfg.video_token_id}
        is_mm = torch.tensor([t in mm_ids for t in seq[:L]] + [False] * (L - len(seq[:L])), dtype=torch.bool, device=dev)
        proj = lambda name: self.text_projection(info[name].to(dev, self.dtype_).reshape(1, -1))
        pad, bos, eos = proj("tts_pad_embed"), proj("tts_bos_embed"), proj("tts_eos_embed")
        codec = self.decoder.embed_tokens
        special = torch.tensor([cfg.codec_nothink_id, cfg.codec_think_bos_id, cfg.codec_think_eos_id,
                                self.speaker_token(info.get("voice_type") or info.get("voice")), cfg.codec_pad_id,
                                cfg.codec_bos_id], device=dev) % codec.shape[0]
        codec_rows = codec[special]                                          # [6, Dt]

        def user_part(a, b):
            if b <= a:
                return emb.new_zeros(0, pad.shape[1])
            text = self.text_projection(emb[a:b].contiguous())
            m = is_mm[a:b]
            if bool(m.any()):
                text = torch.where(m[:, None], self.hidden_projection(hid[a:b].contiguous()), text)
            return text

        streaming = bool(info.get("thinker_stream"))

        def assistant_part(a, header):
            """a: first row of the turn; header: number of ChatML header rows (3, or 0 without ChatML)."""
            h = self.text_projection(emb[a:L].contiguous()) if L > a else emb.new_zeros(0, pad.shape[1])
            first = h[header:header + 1] if h.shape[0] > header else torch.zeros_like(pad)
            text = torch.cat([h[:header], pad.expand(4, -1), bos, first], dim=0)
            text[header:] += codec_rows
            if streaming:                     # the reply is still growing: no end marker yet
                return text, h[header + 1:].contiguous()
            trailing = torch.cat([h[header + 1:], eos], dim=0) if h.shape[0] > header + 1 else torch.zeros_like(eos)
            return text, trailing

        starts = [i for i, t in enumerate(prompt_ids[:n_in]) if t == cfg.im_start_token_id] + [L]
        parts, trailing = [], None
        if len(starts) > 1 and starts[0] > 0:
            parts.append(user_part(0, starts[0]))                            # tokens before the first turn
        for i in range(len(starts) - 1):
            a, b = starts[i], starts[i + 1]
            role = prompt_ids[a + 1] if a + 1 < n_in else None
            last = i == len(starts) - 2
            if role == cfg.system_token_id or (role == cfg.assistant_token_id and not last):
                continue
            if role == cfg.assistant_token_id:
                text, trailing = assistant_part(a, 3)
                parts.append(text)
            else:
                parts.append(user_part(a, min(b, n_in) if last else b))
        if trailing is None:
            # no ChatML assistant header in the prompt: the whole prompt is context, the reply starts
            # with the first generated token
            if len(starts) == 1:
                parts.append(user_part(0, n_in))
            text, trailing = assistant_part(n_in, 0)
            parts.append(text)
        head = torch.cat(parts, dim=0).contiguous()
        req.prompt_embeds = head
        req.prompt_token_ids = [0] * head.shape[0]
        req.runtime_state.update(text_steps=trailing, tts_pad=pad, frames=[], next_embed=None, stream_open=streaming,
                                 tts_eos=eos, pending=None)

    @torch.no_grad()
    def on_stream_update(self, req, payload: dict) -> None:
        """More reply rows of a thinker that is still running (``thinker_embeddings`` [n, D_thinker], may be
        empty) and / or the news that it has finished.  A request that was waiting for its next row goes on."""
        st = req.runtime_state
        if not st.get("stream_open"):
            return
        dev = self.decoder.embed_tokens.device
        rows = payload.get("thinker_embeddings")
        ts = st["text_steps"]
        if rows is not None and rows.shape[0]:
            ts = torch.cat([ts, self.text_projection(rows.to(dev, self.dtype_).contiguous())], dim=0)
        if payload.get("finished"):
            ts = torch.cat([ts, st["tts_eos"]], dim=0) if ts.shape[0] else torch.zeros_like(st["tts_eos"])
            st["stream_open"] = False
        st["text_steps"] = ts
        if req.decode_blocked and st.get("pending") is not None:
            k, base = st["pending"]
            if k < ts.shape[0]:
                st["next_embed"] = base + ts[k:k + 1]
            elif not st["stream_open"]:
                st["next_embed"] = base + st["tts_pad"]
            else:
                return
            st["pending"] = None
            req.decode_blocked = False

    def input_embeds_for(self, req, start, n):
        if start < req.num_prompt_tokens:
            return req.prompt_embeds[start:start + n]
        ne = req.runtime_state.get("next_embed")
        return ne if ne is not None else None

    def compute_logits(self, hidden):
        return self.codec_head(hidden)

    @torch.no_grad()
    def postprocess_sampled(self, reqs, ids, hidden):
        """Complete each sampled code 0 to a full frame with the code predictor and prepare the
        next step's input embedding."""
        codec = self.decoder.embed_tokens
        code0 = ids.long().clamp(0, codec.shape[0] - 1)
        e0 = codec[code0]
        temp = max((r.sampling_params.temperature for r in reqs), default=0.0)
        seed = reqs[0].sampling_params.seed or 0
        rest, summed = self.code_predictor.generate(hidden.to(self.dtype_), e0, temperature=temp, seed=seed,
                                                    step=len(reqs[0].output_token_ids))
        frames = torch.cat([code0[:, None], rest], dim=1)                     # [n, G]
        for i, r in enumerate(reqs):
            st = r.runtime_state
            k = len(r.output_token_ids)                                      # index of this frame
            ts = st.get("text_steps")
            nxt = e0[i:i + 1] + summed[i:i + 1]
            if ts is not None and k >= ts.shape[0] and st.get("stream_open"):
                # the thinker has not produced this step's reply row yet: wait for it
                st["pending"], st["next_embed"] = (k, nxt), None
                r.decode_blocked = True
            else:
                text = ts[k:k + 1] if ts is not None and k < ts.shape[0] else st.get("tts_pad")
                st["next_embed"] = nxt + text if text is not None else nxt
            r.multimodal_outputs.setdefault("codes", []).append(frames[i:i + 1])
        return ids

    @torch.no_grad()
    def load_weights(self, weights):
        """Checkpoint names under ``talker.``: ``model.*`` (decoder, ``model.codec_embedding`` is its
        embedding table), ``text_projection.*``, ``hidden_projection.*``, ``codec_head.weight``,
        ``code_predictor.*``.  Names of other stages are ignored."""
        groups = {"model.": [], "text_projection.": [], "hidden_projection.": [], "code_predictor.": []}
        loaded = set()
        for n, w in weights:
            if n.startswith(("thinker.", "code2wav.")):
                continue
            full = n
            n = n[len("talker."):] if n.startswith("talker.") else n
            if n == "codec_head.weight":
                self.codec_head.weight.copy_(w.to(self.codec_head.weight.dtype))
                loaded.add(full)
                continue
            for pre, lst in groups.items():
                if n.startswith(pre):
                    lst.append((n if pre == "model." else n[len(pre):], w, full))
                    break
        subs = {"model.": self.decoder, "text_projection.": self.text_projection,
                "hidden_projection.": self.hidden_projection, "code_predictor.": self.code_predictor}
        for pre, lst in groups.items():
            names = {n: full for n, _, full in lst}
            got = subs[pre].load_weights([(n, w) for n, w, _ in lst])
            loaded |= {names[n] for n in got}
        return loaded
