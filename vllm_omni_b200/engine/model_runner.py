"""Model runners of the AR engine.

``ARModelRunner``: turns a ``SchedulerOutput`` into one flattened batch (prefill segments +
decode tokens), runs the stage model on the paged KV cache, samples on the device and hands
per-request multimodal outputs (hidden states of captured layers, codec codes ...) to the
engine as DEVICE tensors — the reference copies hidden states to the CPU every step
(vllm_omni/worker/gpu_ar_model_runner.py:525-568).  It also extracts KV pages for stage
hand-off (vllm_omni/distributed/omni_connectors/kv_transfer_manager.py:217-276).

``GenerationModelRunner``: non-autoregressive stages (code2wav, TTS decoders): one forward per
request, outputs returned as multimodal tensors, no sampling
(vllm_omni/worker/gpu_generation_model_runner.py:80-446).
"""
from __future__ import annotations

import os
import zlib

import torch

from ..models.qwen_decoder import ModelBatch, PrefillSeg
from ..ops import kv_cache as KC
from ..ops.sampler import RowParams, sample
from .scheduler import SchedulerOutput


class ARModelRunner:
    def __init__(self, model, device, dtype, num_blocks: int, block_size: int):
        self.model, self.device, self.dtype = model, device, dtype
        self.block_size = block_size
        dec = model.decoder_config
        # under tensor parallelism a rank keeps the pages of its own KV heads only
        kvh = getattr(getattr(model, "decoder", None), "kv_heads_local", dec.num_key_value_heads)
        self.kv_caches = [(torch.zeros(num_blocks, block_size, kvh, dec.head_dim, dtype=dtype, device=device),
                           torch.zeros(num_blocks, block_size, kvh, dec.head_dim, dtype=dtype, device=device))
                          for _ in range(dec.num_hidden_layers)]
        self.tp_group = None        # set by OmniLLM: sampled ids of every step come from rank 0
        # decode-only steps replay a captured graph per batch-size bucket (on by default on a GPU,
        # ``OMNI_AR_CUDA_GRAPH=0`` switches it off); contexts longer than ``OMNI_AR_GRAPH_MAX_TOKENS``
        # (default 4096) and mixed prefill/decode steps run eagerly
        self.graph_runner = None
        on = os.environ.get("OMNI_AR_CUDA_GRAPH", "1" if torch.device(device).type == "cuda" else "0") == "1"
        if on and hasattr(model, "decoder"):
            from .graph_runner import DecodeGraphRunner
            max_tokens = int(os.environ.get("OMNI_AR_GRAPH_MAX_TOKENS", "4096"))
            self.graph_runner = DecodeGraphRunner(model.decoder, self.kv_caches, max(1, max_tokens // block_size),
                                                  capture_layers=getattr(model, "capture", ()))

    # ------------------------------------------------------------------ batch assembly
    def _build_batch(self, sched: SchedulerOutput, kv_mgr):
        ids, pos, slots, prefills = [], [], [], []
        dec_rows, dec_tables, dec_lens = [], [], []
        embeds, emask = [], []
        any_embeds = False
        row = 0
        sample_rows, sample_reqs = [], []
        max_blocks = 1
        for s in sched.scheduled:
            r = s.request
            toks = r.token_slice(s.start, s.num_new_tokens)
            if len(toks) < s.num_new_tokens:            # decode of a request without tokens yet (talker)
                toks = toks + [0] * (s.num_new_tokens - len(toks))
            ids.extend(toks)
            p = self.model.positions_for(r, s.start, s.num_new_tokens)
            pos.append(p)
            slots.extend(kv_mgr.slot_mapping(r, s.start, s.num_new_tokens))
            bt = torch.tensor(r.block_ids, dtype=torch.int32)
            if s.is_prefill:
                prefills.append(PrefillSeg(row, s.num_new_tokens, s.start, bt))
            else:
                dec_rows.append(row)
                dec_tables.append(r.block_ids)
                dec_lens.append(s.start + 1)
                max_blocks = max(max_blocks, len(r.block_ids))
            e = self.model.input_embeds_for(r, s.start, s.num_new_tokens)
            if e is not None:
                any_embeds = True
                embeds.append((row, e))
            if s.samples:
                sample_rows.append(row + s.num_new_tokens - 1)
                sample_reqs.append(r)
            row += s.num_new_tokens
        dev = self.device
        T = row
        positions = torch.cat([p.reshape(-1, p.shape[-1]) if p.dim() > 1 else p[None] for p in pos], dim=-1)
        positions = positions[0] if positions.shape[0] == 1 else positions
        batch = ModelBatch(torch.tensor(ids, dtype=torch.long, device=dev), positions.to(dev),
                           torch.tensor(slots, dtype=torch.int32, device=dev))
        for seg in prefills:
            seg.block_table = seg.block_table.to(dev)
        batch.prefills = prefills
        if dec_rows:
            batch.decode_rows = torch.tensor(dec_rows, dtype=torch.long, device=dev)
            batch.decode_block_tables = torch.tensor([t + [0] * (max_blocks - len(t)) for t in dec_tables],
                                                     dtype=torch.int32, device=dev)
            batch.decode_seq_lens = torch.tensor(dec_lens, dtype=torch.int32, device=dev)
        if any_embeds:
            D = self.model.decoder_config.hidden_size
            buf = torch.zeros(T, D, dtype=self.dtype, device=dev)
            mask = torch.zeros(T, dtype=torch.bool, device=dev)
            for r0, e in embeds:
                buf[r0:r0 + e.shape[0]] = e.to(dev, self.dtype)
                mask[r0:r0 + e.shape[0]] = True
            batch.input_embeds, batch.embeds_mask = buf, mask
        return batch, sample_rows, sample_reqs

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def execute(self, sched: SchedulerOutput, kv_mgr) -> tuple[dict[str, int], list[str]]:
        """Runs one engine step; returns ({request_id: sampled token}, kv_extracted_request_ids)."""
        if sched.empty:
            return {}, []
        batch, sample_rows, sample_reqs = self._build_batch(sched, kv_mgr)
        if self.graph_runner is not None and self.graph_runner.supports(batch):
            hidden, captured = self.graph_runner.run(batch)
        else:
            hidden, captured = self.model.forward_batch(batch, self.kv_caches, sched)
        sampled: dict[str, int] = {}
        if sample_rows:
            rows_t = torch.tensor(sample_rows, dtype=torch.long, device=self.device)
            h = hidden[rows_t].contiguous()
            logits = self.model.compute_logits(h)
            params = [self._row_params(r) for r in sample_reqs]
            ids, _ = sample(logits, params)
            ids = self.model.postprocess_sampled(sample_reqs, ids, h)
            if self.tp_group is not None and self.tp_group.world_size > 1:
                # one request stream on every rank: a rounding difference must not split it
                ids = self.tp_group.broadcast(ids.contiguous(), src=0)
            for r, t in zip(sample_reqs, ids.tolist()):
                sampled[r.request_id] = int(t)
        self.model.collect_outputs(sched, batch, hidden, captured)
        return sampled, []

    def _row_params(self, r) -> RowParams:
        sp = r.sampling_params
        # a process-independent default seed (Python's str hash is salted per process)
        seed = sp.seed if sp.seed is not None else (zlib.crc32(r.request_id.encode()) & 0x7FFFFFFF)
        allowed = sp.extra_args.get("allowed_token_range") if sp.extra_args else None
        pen = sp.repetition_penalty != 1.0 or sp.presence_penalty != 0.0 or sp.frequency_penalty != 0.0
        return RowParams(sp.temperature, sp.top_p, sp.min_p, sp.top_k, sp.repetition_penalty, sp.presence_penalty,
                         sp.frequency_penalty, seed, len(r.output_token_ids), r.all_token_ids if pen else (), r.num_prompt_tokens,
                         list(sp.suppress_token_ids or []), tuple(allowed) if allowed else None)

    # ------------------------------------------------------------------ KV hand-off
    @torch.no_grad()
    def extract_kv(self, request, out_buffers=None) -> dict:
        """Contiguous per-layer K/V of a request ([T, Hkv, D] each).  ``out_buffers`` (a list of
        (k, v) tensors) may point into another stage's peer-mapped memory: the gather kernel
        then IS the transfer."""
        T = request.num_computed_tokens
        bt = torch.tensor(request.block_ids, dtype=torch.int32, device=self.device)
        layers = []
        for li, (kc, vc) in enumerate(self.kv_caches):
            ok, ov = (out_buffers[li] if out_buffers is not None else (None, None))
            layers.append(KC.kv_gather(kc, vc, bt, T, ok, ov))
        return {"num_tokens": T, "layers": layers}


class GenerationModelRunner:
    def __init__(self, model, device, dtype):
        self.model, self.device, self.dtype = model, device, dtype

    @torch.no_grad()
    def execute(self, sched: SchedulerOutput, kv_mgr=None):
        for s in sched.scheduled:
            r = s.request
            out = self.model.generate_for(r, s.start, s.num_new_tokens)
            for k, v in (out or {}).items():
                r.multimodal_outputs.setdefault(k, []).append(v)
        return {}, []
