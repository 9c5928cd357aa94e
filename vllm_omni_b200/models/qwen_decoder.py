"""Decoder-only transformer (Qwen2/Qwen3 family, dense or MoE) on the sm_100a ops, used by
the thinker and talker stages and as a text encoder.

Per layer: RMSNorm -> fused QKV GEMM -> q/k RMSNorm + RoPE in place -> KV pages written ->
attention (tcgen05 flash kernel for prefill segments, paged split-context kernel for decode
tokens) -> output GEMM with the residual add in its epilogue -> RMSNorm -> SwiGLU MLP or
MoE (grouped GEMM) with the residual add fused into the last kernel.

The reference borrows all of this from vLLM (``Qwen3MoeModel``, FusedMoE, paged attention:
vllm_omni/model_executor/models/qwen3_omni/qwen3_omni_moe_thinker.py); checkpoint names
follow the HF layout (``model.layers.N.self_attn.q_proj`` ...) with q/k/v and gate/up stacked
at load time.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
from torch import nn

from ..diffusion.layers.linear import FusedLinear
from ..ops import fused, kv_cache as KC
from ..ops.attention import attention
from ..ops.moe import MoEWorkspace, moe_forward


@dataclass
class DecoderConfig:
    vocab_size: int = 151936
    hidden_size: int = 2048
    num_hidden_layers: int = 48
    num_attention_heads: int = 32
    num_key_value_heads: int = 4
    head_dim: int = 128
    intermediate_size: int = 6144
    num_experts: int = 0                 # 0 = dense MLP
    num_experts_per_tok: int = 8
    moe_intermediate_size: int = 768
    shared_expert_intermediate_size: int = 0   # > 0: a dense SwiGLU expert every token takes, sigmoid-gated
    norm_topk_prob: bool = True
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    qk_norm: bool = True
    attention_bias: bool = False
    mrope_section: tuple | None = None   # e.g. (24, 20, 20): temporal / height / width frequency split
    mrope_interleaved: bool = False
    max_position_embeddings: int = 65536
    tie_word_embeddings: bool = False

    @classmethod
    def from_dict(cls, d: dict) -> "DecoderConfig":
        d = dict(d)
        # newer HF configs nest the rotary settings under "rope_parameters" and call the expert
        # count "num_local_experts"; checkpoints on disk carry either generation of names
        rp = d.get("rope_parameters") or {}
        if "rope_theta" in rp and d.get("rope_theta") is None:
            d["rope_theta"] = float(rp["rope_theta"])
        if d.get("rope_theta") is None:
            d.pop("rope_theta", None)
        if not d.get("num_experts") and d.get("num_local_experts"):
            d["num_experts"] = d["num_local_experts"]
        rs = d.get("rope_scaling") or rp
        if "mrope_section" in rs and "mrope_section" not in d:
            d["mrope_section"] = tuple(rs["mrope_section"])
            d["mrope_interleaved"] = bool(rs.get("mrope_interleaved", rs.get("interleaved", False)))
        if "head_dim" not in d and "hidden_size" in d and "num_attention_heads" in d:
            d["head_dim"] = d["hidden_size"] // d["num_attention_heads"]
        keys = set(cls.__dataclass_fields__)
        return cls(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in d.items() if k in keys})


@dataclass
class PrefillSeg:
    start: int            # first row of this segment in the flattened batch
    length: int           # new tokens in this step
    context: int          # tokens already in the cache
    block_table: torch.Tensor | None = None    # int32 [num_blocks_of_request]


@dataclass
class ModelBatch:
    input_ids: torch.Tensor                    # [T]
    positions: torch.Tensor                    # [T] or [3, T] (MRoPE)
    slot_mapping: torch.Tensor                 # int32 [T]
    prefills: list[PrefillSeg] = field(default_factory=list)
    decode_rows: torch.Tensor | None = None    # int64 [n] rows of decode tokens
    decode_block_tables: torch.Tensor | None = None
    decode_seq_lens: torch.Tensor | None = None
    input_embeds: torch.Tensor | None = None   # [T, D] replaces the embedding lookup where mask is set
    embeds_mask: torch.Tensor | None = None    # bool [T]


class RotaryTable:
    def __init__(self, head_dim: int, theta: float, max_pos: int):
        self.head_dim, self.theta, self.max_pos = head_dim, theta, max_pos
        self.inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
        self._dev = {}

    def cos_sin_for(self, positions: torch.Tensor, mrope_section=None, interleaved=False):
        """Per-token tables [T, head_dim/2] (fp32).  positions: [T] or [3, T]."""
        inv = self._dev.get(positions.device)
        if inv is None:
            inv = self.inv_freq.to(positions.device)
            self._dev[positions.device] = inv
        if positions.dim() == 1:
            ang = positions.float()[:, None] * inv[None, :]
        else:
            ang3 = positions.float()[:, :, None] * inv[None, None, :]          # [3, T, Dh/2]
            if interleaved:
                # frequency i takes its position from axis (i % 3) inside the sectioned range
                ang = ang3[0].clone()
                for ax, off in ((1, 1), (2, 2)):
                    n = mrope_section[ax] * 3
                    ang[:, off:n:3] = ang3[ax][:, off:n:3]
            else:
                parts, o = [], 0
                for ax, n in enumerate(mrope_section):
                    parts.append(ang3[ax][:, o:o + n])
                    o += n
                ang = torch.cat(parts, dim=-1)
        return ang.cos().contiguous(), ang.sin().contiguous()


class DecoderLayer(nn.Module):
    def __init__(self, cfg: DecoderConfig, dtype, device):
        super().__init__()
        D, H, Hkv, Dh = cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        P = lambda *s: nn.Parameter(torch.ones(*s, dtype=dtype, device=device), requires_grad=False)
        self.input_layernorm = P(D)
        self.qkv_proj = FusedLinear(D, (H + 2 * Hkv) * Dh, bias=cfg.attention_bias, dtype=dtype, device=device)
        self.q_norm = P(Dh) if cfg.qk_norm else None
        self.k_norm = P(Dh) if cfg.qk_norm else None
        self.o_proj = FusedLinear(H * Dh, D, bias=False, dtype=dtype, device=device)
        self.post_attention_layernorm = P(D)
        if cfg.num_experts:
            E, F_ = cfg.num_experts, cfg.moe_intermediate_size
            self.router = FusedLinear(D, E, bias=False, dtype=dtype, device=device)
            self.w13 = nn.Parameter(torch.empty(E, 2 * F_, D, dtype=dtype, device=device).normal_(0, 0.02),
                                    requires_grad=False)
            self.w2 = nn.Parameter(torch.empty(E, D, F_, dtype=dtype, device=device).normal_(0, 0.02),
                                   requires_grad=False)
            self.moe_ws = MoEWorkspace()
            Fs = cfg.shared_expert_intermediate_size
            if Fs:
                self.shared_gate_up = FusedLinear(D, 2 * Fs, bias=False, dtype=dtype, device=device)
                self.shared_down = FusedLinear(Fs, D, bias=False, dtype=dtype, device=device)
                self.shared_expert_gate = nn.Parameter(torch.empty(1, D, dtype=dtype, device=device).normal_(0, 0.02),
                                                       requires_grad=False)
        else:
            self.gate_up = FusedLinear(D, 2 * cfg.intermediate_size, bias=False, dtype=dtype, device=device)
            self.down = FusedLinear(cfg.intermediate_size, D, bias=False, dtype=dtype, device=device)


class QwenDecoderModel(nn.Module):
    def __init__(self, cfg: DecoderConfig, dtype=torch.bfloat16, device=None, with_lm_head: bool = True):
        super().__init__()
        self.cfg, self.dtype_ = cfg, dtype
        self.embed_tokens = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device)
                                         .normal_(0, 0.02), requires_grad=False)
        self.layers = nn.ModuleList([DecoderLayer(cfg, dtype, device) for _ in range(cfg.num_hidden_layers)])
        self.norm = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype, device=device), requires_grad=False)
        self.lm_head = None
        if with_lm_head and not cfg.tie_word_embeddings:
            self.lm_head = FusedLinear(cfg.hidden_size, cfg.vocab_size, bias=False, dtype=dtype, device=device)
        self.rope = RotaryTable(cfg.head_dim, cfg.rope_theta, cfg.max_position_embeddings)
        self.ep_group = None          # expert-parallel group: experts sharded, partial outputs summed
        self.ep_range = (0, cfg.num_experts)
        self.ep_reduce = None         # RowParallelReduce over the EP group (peer-memory sum of the partials)
        self.tp_group = None          # tensor-parallel group: heads and MLP columns sharded
        self.tp_reduce = None
        self.local_heads = (cfg.num_attention_heads, cfg.num_key_value_heads)   # (q, kv) heads on this rank

    @property
    def kv_heads_local(self) -> int:
        """KV heads whose pages this rank keeps (all of them without tensor parallelism)."""
        return self.local_heads[1]

    @torch.no_grad()
    def enable_tensor_parallel(self, group, mode: str | None = None, expert_parallel: bool = False) -> None:
        """Shard the decoder over ``group`` (the reference takes this from vLLM's
        ``ColumnParallelLinear`` / ``RowParallelLinear`` / ``FusedMoE`` under ``tensor_parallel_size``,
        vllm_omni/model_executor/stage_configs/qwen3_omni_moe.yaml:27):

        * attention: rank r keeps q heads [r H/P, (r+1) H/P) and the KV heads they read (a KV head is
          replicated when there are fewer KV heads than ranks); ``o_proj`` becomes row-parallel;
        * dense MLP: gate/up column-parallel, down row-parallel;
        * MoE: ``expert_parallel=True`` keeps whole experts per rank, otherwise every expert's FFN
          dimension is sliced; either way each rank produces a partial sum of the MoE output;
        * embeddings, norms, router, shared expert and the LM head stay replicated.

        Row-parallel outputs are summed by ``RowParallelReduce`` (GEMM epilogue stores to the row
        owners + local reduce on the GPU, all-reduce on CPU / ``mode="nccl"``)."""
        from ..parallel.tensor_parallel import RowParallelReduce, shard_cols
        cfg = self.cfg
        P, r = group.world_size, group.rank_in_group
        if P == 1:
            return
        H, Hkv, Dh = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        if H % P:
            raise ValueError(f"num_attention_heads ({H}) must be divisible by tensor_parallel_size ({P})")
        Hl = H // P
        if Hkv % P == 0:
            kv_lo, Hkvl = r * (Hkv // P), Hkv // P
        elif P % Hkv == 0:
            kv_lo, Hkvl = r // (P // Hkv), 1              # several ranks share one KV head
        else:
            raise ValueError(f"num_key_value_heads ({Hkv}) and tensor_parallel_size ({P}) must divide one another")
        self.tp_group = group
        self.tp_reduce = RowParallelReduce(group, mode)
        self.local_heads = (Hl, Hkvl)
        qs = slice(r * Hl * Dh, (r + 1) * Hl * Dh)
        ks = slice(H * Dh + kv_lo * Dh, H * Dh + (kv_lo + Hkvl) * Dh)
        vs = slice((H + Hkv) * Dh + kv_lo * Dh, (H + Hkv) * Dh + (kv_lo + Hkvl) * Dh)

        def relinear(old: FusedLinear, w: torch.Tensor, b: torch.Tensor | None) -> FusedLinear:
            new = FusedLinear(w.shape[1], w.shape[0], bias=b is not None, dtype=w.dtype, device="meta")
            new.weight = nn.Parameter(w.contiguous(), requires_grad=False)
            if b is not None:
                new.bias = nn.Parameter(b.contiguous(), requires_grad=False)
            return new

        for layer in self.layers:
            w = layer.qkv_proj.weight.data
            b = layer.qkv_proj.bias.data if layer.qkv_proj.bias is not None else None
            layer.qkv_proj = relinear(layer.qkv_proj, torch.cat([w[qs], w[ks], w[vs]], 0),
                                      None if b is None else torch.cat([b[qs], b[ks], b[vs]], 0))
            layer.o_proj = relinear(layer.o_proj, layer.o_proj.weight.data[:, qs], None)
            if not cfg.num_experts:
                F_ = cfg.intermediate_size
                if F_ % P:
                    raise ValueError(f"intermediate_size ({F_}) must be divisible by tensor_parallel_size ({P})")
                Fl = F_ // P
                gu = layer.gate_up.weight.data
                layer.gate_up = relinear(layer.gate_up, torch.cat([gu[r * Fl:(r + 1) * Fl],
                                                                   gu[F_ + r * Fl:F_ + (r + 1) * Fl]], 0), None)
                layer.down = relinear(layer.down, shard_cols(layer.down.weight.data, r, P), None)
            elif not expert_parallel:
                F_ = cfg.moe_intermediate_size
                if F_ % (P * 8):
                    raise ValueError(f"moe_intermediate_size ({F_}) must be divisible by 8 x tensor_parallel_size")
                Fl = F_ // P
                w13 = layer.w13.data
                layer.w13 = nn.Parameter(torch.cat([w13[:, r * Fl:(r + 1) * Fl], w13[:, F_ + r * Fl:F_ + (r + 1) * Fl]],
                                                   1).contiguous(), requires_grad=False)
                layer.w2 = nn.Parameter(layer.w2.data[:, :, r * Fl:(r + 1) * Fl].contiguous(), requires_grad=False)
        if cfg.num_experts:
            if expert_parallel:
                self.enable_expert_parallel(group, mode)
            else:
                # FFN-sliced experts: every rank runs all experts on its slice; same partial-sum path
                self.ep_group, self.ep_range, self.ep_reduce = group, (0, cfg.num_experts), self.tp_reduce

    @torch.no_grad()
    def enable_expert_parallel(self, group, mode: str | None = None) -> None:
        """Keep experts [r E/P, (r+1) E/P) on rank r of ``group``.  Tokens are replicated across the
        group (attention is not sharded here), so dispatch is local; the partial sums of the local
        experts are added across ranks either by the combine kernel storing them straight into the
        row owners' peer memory followed by a local reduce (``mode="peer"``) or by an all-reduce
        (``mode="nccl"``, the baseline and the CPU path)."""
        cfg = self.cfg
        P, r = group.world_size, group.rank_in_group
        if not cfg.num_experts or P == 1:
            return
        if cfg.num_experts % P:
            raise ValueError(f"num_experts ({cfg.num_experts}) must be divisible by the expert-parallel size ({P})")
        per = cfg.num_experts // P
        lo, hi = r * per, (r + 1) * per
        for layer in self.layers:
            layer.w13 = nn.Parameter(layer.w13.data[lo:hi].clone(), requires_grad=False)
            layer.w2 = nn.Parameter(layer.w2.data[lo:hi].clone(), requires_grad=False)
        from ..parallel.tensor_parallel import RowParallelReduce
        self.ep_group, self.ep_range = group, (lo, hi)
        self.ep_reduce = RowParallelReduce(group, mode)

    # ------------------------------------------------------------------ forward
    def embed(self, batch: ModelBatch) -> torch.Tensor:
        x = self.embed_tokens[batch.input_ids.long().clamp(0, self.cfg.vocab_size - 1)]
        if batch.input_embeds is not None:
            m = batch.embeds_mask
            x = torch.where(m[:, None], batch.input_embeds.to(x.dtype), x) if m is not None else batch.input_embeds.to(x.dtype)
        return x.contiguous()

    def attention_block(self, layer: DecoderLayer, qkv: torch.Tensor, batch: ModelBatch, k_cache, v_cache, out):
        cfg = self.cfg
        (H, Hkv), Dh = self.local_heads, cfg.head_dim
        T = qkv.shape[0]
        q = qkv[:, :H * Dh].view(T, H, Dh)
        k = qkv[:, H * Dh:(H + Hkv) * Dh].view(T, Hkv, Dh)
        v = qkv[:, (H + Hkv) * Dh:].view(T, Hkv, Dh)
        if k_cache is not None:
            KC.kv_write(k, v, k_cache, v_cache, batch.slot_mapping)
        scale = 1.0 / math.sqrt(Dh)
        o = out.view(T, H, Dh)
        for seg in batch.prefills:
            s, n = seg.start, seg.length
            if seg.context == 0 or k_cache is None:
                attention(q[None, s:s + n], k[None, s:s + n], v[None, s:s + n], scale=scale, causal=True,
                          out=o[None, s:s + n])
            elif q.is_cuda and KC.tma_pages_ok(k_cache.shape[1], Dh):
                # chunked prefill straight from the pages (this chunk's K/V were written above)
                KC.paged_prefill(q[s:s + n], k_cache, v_cache, seg.block_table, seg.context + n, scale=scale,
                                 out=o[s:s + n])
            else:
                gk, gv = KC.kv_gather(k_cache, v_cache, seg.block_table, seg.context + n)
                attention(q[None, s:s + n], gk[None], gv[None], scale=scale, causal=True, q_offset=seg.context,
                          out=o[None, s:s + n])
        if batch.decode_rows is not None and batch.decode_rows.numel():
            rows = batch.decode_rows
            if not batch.prefills and rows.numel() == T and q.is_cuda:
                # a decode-only step: the rows ARE the batch in order; read q and write o in place
                KC.paged_decode(q, k_cache, v_cache, batch.decode_block_tables, batch.decode_seq_lens, scale=scale, out=o)
            else:
                qd = q[rows].contiguous()
                od = KC.paged_decode(qd, k_cache, v_cache, batch.decode_block_tables, batch.decode_seq_lens, scale=scale)
                o[rows] = od
        return out

    def forward(self, batch: ModelBatch, kv_caches=None, capture_layers=(), deepstack=None):
        """Returns (hidden [T, D] after the final norm, captured layer outputs).  ``deepstack``: list
        of [T, D] tensors; entry i is added to the output of layer i (visual features of the
        vision tower's intermediate blocks, zero on the other rows)."""
        cfg = self.cfg
        (H, Hkv), Dh = self.local_heads, cfg.head_dim        # this rank's heads under tensor parallelism
        x = self.embed(batch)
        T = x.shape[0]
        cos, sin = self.rope.cos_sin_for(batch.positions, cfg.mrope_section, cfg.mrope_interleaved)
        captured = {}
        if 0 in capture_layers:
            captured[0] = x.clone()
        xn = torch.empty_like(x)
        attn = torch.empty(T, H * Dh, dtype=x.dtype, device=x.device)
        tp_cap = max(64, 1 << (T - 1).bit_length())          # peer-buffer bucket of the row-parallel reduces
        for li, layer in enumerate(self.layers):
            fused.norm_modulate(x, weight=layer.input_layernorm, rms=True, eps=cfg.rms_norm_eps, out=xn)
            qkv = layer.qkv_proj(xn)
            fused.qk_norm_rope_(qkv.view(1, T, -1), H, Hkv, Dh, wq=layer.q_norm, wk=layer.k_norm, cos=cos, sin=sin,
                                interleaved=False, eps=cfg.rms_norm_eps)
            kc, vc = kv_caches[li] if kv_caches is not None else (None, None)
            self.attention_block(layer, qkv, batch, kc, vc, attn)
            if self.tp_reduce is not None:
                self.tp_reduce.linear(layer.o_proj, attn, residual=x, out=x, capacity=tp_cap)   # sum over ranks
            else:
                layer.o_proj(attn, residual=x, out=x)
            fused.norm_modulate(x, weight=layer.post_attention_layernorm, rms=True, eps=cfg.rms_norm_eps, out=xn)
            if cfg.num_experts:
                logits = layer.router(xn)
                e_lo, e_hi = self.ep_range
                shared = None
                if cfg.shared_expert_intermediate_size:
                    # replicated under expert parallelism: added once, after the routed experts
                    g = torch.sigmoid(xn.float() @ layer.shared_expert_gate.float().t())
                    shared = layer.shared_down(fused.silu_mul(layer.shared_gate_up(xn))).float().mul_(g)
                if self.ep_group is None or self.ep_group.world_size == 1:
                    moe_forward(xn, logits, layer.w13, layer.w2, cfg.num_experts_per_tok, cfg.norm_topk_prob,
                                ws=layer.moe_ws, residual=x, out=x)
                elif self.ep_reduce is not None and self.ep_reduce.mode == "peer" and x.is_cuda:
                    # combine stores each token's partial sum into its row owner's peer slot; the
                    # owners reduce locally, add the residual and push the rows to every rank
                    cap = max(64, 1 << (T - 1).bit_length())
                    res = self.ep_reduce.reduce_from(
                        lambda per, ptrs: moe_forward(xn, logits, layer.w13, layer.w2, cfg.num_experts_per_tok,
                                                      cfg.norm_topk_prob, e_lo=e_lo, e_hi=e_hi, ws=layer.moe_ws,
                                                      scatter=(per, ptrs)),
                        T, cfg.hidden_size, x.dtype, x.device, residual=x, capacity=cap)
                    x.copy_(res)
                else:
                    part = moe_forward(xn, logits, layer.w13, layer.w2, cfg.num_experts_per_tok, cfg.norm_topk_prob,
                                       e_lo=e_lo, e_hi=e_hi, ws=layer.moe_ws)
                    self.ep_group.all_reduce(part)
                    x.add_(part)
                if shared is not None:
                    x.add_(shared.to(x.dtype))
            else:
                h = fused.silu_mul(layer.gate_up(xn))
                if self.tp_reduce is not None:
                    self.tp_reduce.linear(layer.down, h, residual=x, out=x, capacity=tp_cap)
                else:
                    layer.down(h, residual=x, out=x)
            if deepstack is not None and li < len(deepstack):
                x.add_(deepstack[li].to(x.dtype))
            if (li + 1) in capture_layers:
                captured[li + 1] = x.clone()
        hidden = fused.norm_modulate(x, weight=self.norm, rms=True, eps=cfg.rms_norm_eps)
        return hidden, captured

    def compute_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        if self.lm_head is not None:
            return self.lm_head(hidden)
        from ..ops.gemm import linear
        return linear(hidden, self.embed_tokens)

    # ------------------------------------------------------------------ weights
    @torch.no_grad()
    def load_weights(self, weights, prefix: str = "model.") -> set:
        cfg = self.cfg
        H, Hkv, Dh = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        F_ = cfg.moe_intermediate_size if cfg.num_experts else cfg.intermediate_size
        loaded = set()
        for name, w in weights:
            n = name[len(prefix):] if name.startswith(prefix) else name
            tgt, sl = None, None
            if n in ("embed_tokens.weight", "codec_embedding.weight"):   # the talker calls its table codec_embedding
                tgt = self.embed_tokens
            elif n == "norm.weight":
                tgt = self.norm
            elif name in ("lm_head.weight", prefix + "lm_head.weight") and self.lm_head is not None:
                tgt = self.lm_head.weight
            elif n.startswith("layers."):
                parts = n.split(".")
                layer = self.layers[int(parts[1])]
                rest = ".".join(parts[2:])
                qkv_off = {"self_attn.q_proj": (0, H * Dh), "self_attn.k_proj": (H * Dh, (H + Hkv) * Dh),
                           "self_attn.v_proj": ((H + Hkv) * Dh, (H + 2 * Hkv) * Dh)}
                for k, (a, b) in qkv_off.items():
                    if rest == k + ".weight":
                        tgt, sl = layer.qkv_proj.weight, (a, b)
                    elif rest == k + ".bias" and layer.qkv_proj.bias is not None:
                        tgt, sl = layer.qkv_proj.bias, (a, b)
                simple = {"input_layernorm.weight": layer.input_layernorm,
                          "post_attention_layernorm.weight": layer.post_attention_layernorm,
                          "self_attn.o_proj.weight": layer.o_proj.weight,
                          "self_attn.q_norm.weight": layer.q_norm, "self_attn.k_norm.weight": layer.k_norm}
                if rest in simple and simple[rest] is not None:
                    tgt = simple[rest]
                if cfg.num_experts:
                    if rest == "mlp.gate.weight":
                        tgt = layer.router.weight
                    elif rest == "mlp.experts.gate_up_proj":        # experts stacked: [E, 2F, D]
                        tgt = layer.w13
                    elif rest == "mlp.experts.down_proj":           # [E, D, F]
                        tgt = layer.w2
                    elif cfg.shared_expert_intermediate_size and rest.startswith("mlp.shared_expert"):
                        Fs = cfg.shared_expert_intermediate_size
                        if rest == "mlp.shared_expert.gate_proj.weight":
                            tgt, sl = layer.shared_gate_up.weight, (0, Fs)
                        elif rest == "mlp.shared_expert.up_proj.weight":
                            tgt, sl = layer.shared_gate_up.weight, (Fs, 2 * Fs)
                        elif rest == "mlp.shared_expert.down_proj.weight":
                            tgt = layer.shared_down.weight
                        elif rest == "mlp.shared_expert_gate.weight":
                            tgt = layer.shared_expert_gate
                    elif rest.startswith("mlp.experts."):
                        e = int(parts[4])
                        kind = parts[5]
                        if kind == "gate_proj":
                            tgt, sl = layer.w13[e], (0, F_)
                        elif kind == "up_proj":
                            tgt, sl = layer.w13[e], (F_, 2 * F_)
                        elif kind == "down_proj":
                            tgt = layer.w2[e]
                else:
                    if rest == "mlp.gate_proj.weight":
                        tgt, sl = layer.gate_up.weight, (0, F_)
                    elif rest == "mlp.up_proj.weight":
                        tgt, sl = layer.gate_up.weight, (F_, 2 * F_)
                    elif rest == "mlp.down_proj.weight":
                        tgt = layer.down.weight
            if tgt is None:
                continue
            dst = tgt if sl is None else tgt[sl[0]:sl[1]]
            dst.copy_(w.to(dst.dtype).reshape(dst.shape))
            loaded.add(name)
        return loaded


def reference_forward(model: QwenDecoderModel, input_ids: torch.Tensor, positions: torch.Tensor | None = None):
    """Plain PyTorch fp32 forward of one full sequence (no cache): the engine's oracle."""
    import torch.nn.functional as F
    cfg = model.cfg
    H, Hkv, Dh = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    T = input_ids.numel()
    f = lambda t: t.float()
    x = f(model.embed_tokens)[input_ids.long()]
    pos = torch.arange(T, device=input_ids.device) if positions is None else positions
    cos, sin = model.rope.cos_sin_for(pos, cfg.mrope_section, cfg.mrope_interleaved)
    rms = lambda t, w: t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * f(w)
    for layer in model.layers:
        xn = rms(x, layer.input_layernorm)
        qkv = F.linear(xn, f(layer.qkv_proj.weight), None if layer.qkv_proj.bias is None else f(layer.qkv_proj.bias))
        q = qkv[:, :H * Dh].view(T, H, Dh)
        k = qkv[:, H * Dh:(H + Hkv) * Dh].view(T, Hkv, Dh)
        v = qkv[:, (H + Hkv) * Dh:].view(T, Hkv, Dh)
        if layer.q_norm is not None:
            q, k = rms(q, layer.q_norm), rms(k, layer.k_norm)
        q = fused.apply_rope_reference(q, cos, sin, False)
        k = fused.apply_rope_reference(k, cos, sin, False)
        kk = k.repeat_interleave(H // Hkv, dim=1)
        vv = v.repeat_interleave(H // Hkv, dim=1)
        s = torch.einsum("qhd,khd->hqk", q, kk) / math.sqrt(Dh)
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool, device=s.device), 1)[None], float("-inf"))
        o = torch.einsum("hqk,khd->qhd", s.softmax(-1), vv).reshape(T, H * Dh)
        x = x + F.linear(o, f(layer.o_proj.weight))
        xn = rms(x, layer.post_attention_layernorm)
        if cfg.num_experts:
            logits = F.linear(xn, f(layer.router.weight))
            p = logits.softmax(-1)
            w, ids = torch.topk(p, cfg.num_experts_per_tok, dim=-1)
            if cfg.norm_topk_prob:
                w = w / w.sum(-1, keepdim=True)
            y = torch.zeros_like(x)
            Fd = cfg.moe_intermediate_size
            for t in range(T):
                for j in range(cfg.num_experts_per_tok):
                    e = int(ids[t, j])
                    h = F.linear(xn[t], f(layer.w13[e]))
                    y[t] += w[t, j] * F.linear(F.silu(h[:Fd]) * h[Fd:], f(layer.w2[e]))
            if cfg.shared_expert_intermediate_size:
                Fs = cfg.shared_expert_intermediate_size
                h = F.linear(xn, f(layer.shared_gate_up.weight))
                y = y + torch.sigmoid(F.linear(xn, f(layer.shared_expert_gate))) * \
                    F.linear(F.silu(h[:, :Fs]) * h[:, Fs:], f(layer.shared_down.weight))
            x = x + y
        else:
            h = F.linear(xn, f(layer.gate_up.weight))
            Fd = cfg.intermediate_size
            x = x + F.linear(F.silu(h[:, :Fd]) * h[:, Fd:], f(layer.down.weight))
    return rms(x, model.norm)
