"""AR engine: request intake, scheduling loop, output assembly.

One ``LLMEngine`` serves one stage.  ``add_request`` accepts text / token / embedding
prompts (tensors in ``additional_information`` stay tensors — the reference serialises them to
bytes to cross its engine-core process boundary, vllm_omni/engine/input_processor.py:260-281);
``step`` runs one scheduler + model-runner iteration and returns ``RequestOutput`` records:
incremental ones for streaming and a final one per request that carries the accumulated
multimodal tensors (the role of vllm_omni/engine/output_processor.py).
"""
from __future__ import annotations

import os
import time

import torch

from ..inputs.data import SamplingParams
from ..logger import init_logger
from ..outputs import CompletionOutput, RequestOutput
from .kv_cache_manager import KVCacheManager
from .model_runner import ARModelRunner, GenerationModelRunner
from .request import FINISH_REASON, Request, RequestStatus
from .scheduler import OmniARScheduler, OmniGenerationScheduler
from .tokenizer import ByteTokenizer, IncrementalDetokenizer, get_tokenizer

logger = init_logger(__name__)


class LLMEngine:
    def __init__(self, model, tokenizer=None, device=None, dtype=torch.bfloat16, block_size: int = 16,
                 num_gpu_blocks: int | None = None, gpu_memory_utilization: float = 0.9, max_num_seqs: int = 64,
                 max_num_batched_tokens: int = 8192, max_model_len: int = 32768, kv_transfer_criteria=None,
                 chunk_adapter=None, kv_transfer_manager=None, stage_id: int = 0, engine_output_type: str | None = None):
        self.model = model
        self.device = torch.device(device) if device is not None else torch.device(
            "cuda" if torch.cuda.is_available() else "cpu")
        self.dtype = dtype
        self.max_num_batched_tokens = max_num_batched_tokens
        self.tokenizer = tokenizer or get_tokenizer(None)
        if hasattr(model, "text_tokenizer"):             # models that tokenize request fields themselves (TTS instructions)
            model.text_tokenizer = self.tokenizer
        self.stage_id = stage_id
        self.engine_output_type = engine_output_type or getattr(model, "engine_output_type", "text")
        self.generation = bool(getattr(model, "is_generation_model", False))
        dec = getattr(model, "decoder_config", None)
        if self.generation or dec is None:
            self.kv = KVCacheManager(1, block_size)
            self.runner = GenerationModelRunner(model, self.device, dtype)
            self.scheduler = OmniGenerationScheduler(self.kv, max_num_seqs, max(max_num_batched_tokens, 1 << 20),
                                                     chunk_adapter=chunk_adapter)
        else:
            if num_gpu_blocks is None:
                num_gpu_blocks = self._profile_num_blocks(dec, block_size, gpu_memory_utilization, max_model_len,
                                                          max_num_seqs)
            self.kv = KVCacheManager(num_gpu_blocks, block_size)
            self.runner = ARModelRunner(model, self.device, dtype, num_gpu_blocks, block_size)
            self.scheduler = OmniARScheduler(self.kv, max_num_seqs, max_num_batched_tokens, kv_transfer_criteria,
                                             chunk_adapter)
        self.kv_transfer_manager = kv_transfer_manager
        self.max_model_len = max_model_len
        self._detok: dict[str, IncrementalDetokenizer] = {}
        self._reqs: dict[str, Request] = {}
        self._errors: list[RequestOutput] = []
        # Steps between progress reports of a running request: 1 = every step (a stage whose output is streamed
        # to the client), n > 1 = every n generated tokens (a stage whose frames feed a chunked consumer),
        # 0 = only the finished request is reported (a stage nobody watches while it runs).
        self.stream_interval = 1
        # Tensors among the progress reports (the model's ``stream_output_keys``) ride only on every n-th generated
        # token of a request; in between they accumulate.  Token ids and text still ride on every report.
        self.stream_mm_interval = 1

    def _activation_reserve(self, dec) -> int:
        rows = int(getattr(self, "max_num_batched_tokens", 8192) or 8192)
        es = torch.empty(0, dtype=self.dtype).element_size()
        D = dec.hidden_size
        per_row = 12 * D + 4 * max(dec.intermediate_size or 0, (dec.num_experts_per_tok or 0) * (dec.moe_intermediate_size or 0))
        if dec.num_experts:
            per_row += 2 * (dec.num_experts_per_tok or 1) * (2 * D + 3 * (dec.moe_intermediate_size or 0))   # two token buckets live
        return int(rows * per_row * es) + (2 << 30)

    def _profile_num_blocks(self, dec, block_size, util, max_model_len, max_num_seqs) -> int:
        per_block = 2 * dec.num_hidden_layers * block_size * dec.num_key_value_heads * dec.head_dim * \
            torch.empty(0, dtype=self.dtype).element_size()
        if self.device.type == "cuda":
            from ..utils.gpu_memory import kv_cache_budget
            free, total = torch.cuda.mem_get_info(self.device)
            # per-process accounting: stages that share this GPU may be initialising concurrently
            budget = kv_cache_budget(total, free, util, self.device.index or 0)
            # the share covers the stage's activations too (prefill scratch of max_num_batched_tokens rows,
            # MoE dispatch buffers, logits of the sampled rows, library workspaces): leave room for them
            budget = max(0, budget - self._activation_reserve(dec))
        else:
            budget = 256 << 20
        want = (max_model_len // block_size + 1) * max_num_seqs
        return int(max(16, min(want, budget // max(per_block, 1))))

    # ------------------------------------------------------------------ intake
    def add_request(self, request_id: str, prompt, sampling_params: SamplingParams | None = None) -> Request:
        sp = sampling_params or SamplingParams()
        text, ids, embeds, info, mm = None, None, None, {}, None
        expects_chunks = False
        if isinstance(prompt, str):
            text = prompt
        elif isinstance(prompt, dict):
            text = prompt.get("prompt")
            ids = prompt.get("prompt_token_ids")
            embeds = prompt.get("prompt_embeds")
            info = dict(prompt.get("additional_information") or {})
            mm = prompt.get("multi_modal_data")
            expects_chunks = bool(info.pop("__expects_chunks__", False))
        else:
            raise TypeError(f"unsupported prompt type {type(prompt)!r}")
        if ids is None:
            if text is not None:
                special = getattr(self.model, "special_token_map", None)
                if special and isinstance(self.tokenizer, ByteTokenizer):
                    # no checkpoint tokenizer (random-weight runs): the model's chat markers and multimodal
                    # placeholders still have to arrive as their single ids
                    ids = self.tokenizer.encode(text, special=special() if callable(special) else special)
                else:
                    ids = self.tokenizer.encode(text)
            elif embeds is not None:
                ids = [0] * embeds.shape[0]
            else:
                ids = []
        if len(ids) > self.max_model_len:
            raise ValueError(f"prompt of {len(ids)} tokens exceeds max_model_len {self.max_model_len}")
        eos = self.model.eos_token_id() if hasattr(self.model, "eos_token_id") else None
        if eos is None:
            eos = getattr(self.tokenizer, "eos_token_id", None)
        req = Request(request_id, list(ids), sp, prompt=text, prompt_embeds=embeds, additional_information=info,
                      multi_modal_data=mm, eos_token_id=eos, expects_more_chunks=expects_chunks)
        if hasattr(self.model, "preprocess_request"):
            self.model.preprocess_request(req)
        self._reqs[request_id] = req
        if sp.detokenize and self.engine_output_type == "text":
            self._detok[request_id] = IncrementalDetokenizer(self.tokenizer, sp.skip_special_tokens)
        self.scheduler.add_request(req)
        return req

    def abort_request(self, request_ids) -> None:
        if isinstance(request_ids, str):
            request_ids = [request_ids]
        for r in self.scheduler.abort(request_ids):
            self._reqs.pop(r.request_id, None)
            self._detok.pop(r.request_id, None)

    def has_unfinished_requests(self) -> bool:
        return self.scheduler.has_unfinished() or bool(self._errors)

    def get_request(self, request_id: str) -> Request | None:
        return self._reqs.get(request_id)

    # ------------------------------------------------------------------ loop
    def _timing(self):
        """Per-phase wall time of the engine loop (``OMNI_ENGINE_TIMING=1``; the device is synchronised at
        the phase boundaries, so use it for diagnosis, not while benchmarking).  Printed at exit."""
        if getattr(self, "_phase", None) is None:
            import atexit
            import json
            import sys
            self._phase = {"steps": 0, "schedule": 0.0, "execute": 0.0, "update": 0.0, "outputs": 0.0, "tokens": 0,
                           "decode_only_steps": 0}
            name = type(self.model).__name__
            atexit.register(lambda: print(json.dumps({"engine_timing": name, **{k: (round(v, 3) if isinstance(v, float) else v)
                                                                              for k, v in self._phase.items()}}),
                                          file=sys.stderr, flush=True))
        return self._phase

    def step(self) -> list[RequestOutput]:
        if os.environ.get("OMNI_ENGINE_TIMING") == "1":
            return self._timed_step()
        return self._step()

    def _timed_step(self) -> list[RequestOutput]:
        ph = self._timing()
        sync = (lambda: torch.cuda.synchronize(self.device)) if self.device.type == "cuda" else (lambda: None)
        outs, self._errors = self._errors, []
        t0 = time.perf_counter()
        sched = self.scheduler.schedule()
        t1 = time.perf_counter()
        ph["schedule"] += t1 - t0
        if sched.empty:
            if self.scheduler.has_unfinished() and not self.scheduler.has_schedulable():
                time.sleep(0.001)
            return outs
        sampled, kv_done = self.runner.execute(sched, self.kv)
        sync()
        t2 = time.perf_counter()
        ph["execute"] += t2 - t1
        ph["steps"] += 1
        ph["tokens"] += sum(s.num_new_tokens for s in sched.scheduled)
        ph["decode_only_steps"] += int(all(s.num_new_tokens == 1 for s in sched.scheduled))
        touched = self.scheduler.update_from_output(sched, sampled, kv_done)
        t3 = time.perf_counter()
        ph["update"] += t3 - t2
        outs += self._finish_step(sched, touched)
        ph["outputs"] += time.perf_counter() - t3
        return outs

    def _step(self) -> list[RequestOutput]:
        outs, self._errors = self._errors, []
        sched = self.scheduler.schedule()
        if sched.empty:
            if self.scheduler.has_unfinished() and not self.scheduler.has_schedulable():
                time.sleep(0.001)          # everything is parked waiting for input chunks
            return outs
        sampled, kv_done = self.runner.execute(sched, self.kv)
        touched = self.scheduler.update_from_output(sched, sampled, kv_done)
        return outs + self._finish_step(sched, touched)

    def _finish_step(self, sched, touched) -> list[RequestOutput]:
        outs: list[RequestOutput] = []
        if sched.kv_transfer_ids and self.kv_transfer_manager is not None:
            done = self.kv_transfer_manager.handle_finished_requests_kv_transfer(
                [self._reqs[r] for r in sched.kv_transfer_ids if r in self._reqs], self.runner)
            self.scheduler.update_from_output(type(sched)(), {}, done)
        elif sched.kv_transfer_ids:
            # a hand-off criterion without a transfer manager: nothing will ever extract the KV
            self.scheduler.update_from_output(type(sched)(), {}, list(sched.kv_transfer_ids))
        now = time.time()
        every = self.stream_interval
        for req in touched:
            if req.first_token_time is None:
                req.first_token_time = now
            if every != 1 and not req.is_finished() and (every <= 0 or len(req.output_token_ids) % every):
                continue        # unreported progress rides in the next report: nothing is marked as sent
            outs.append(self._make_output(req))
            if req.is_finished():
                self._reqs.pop(req.request_id, None)
                self._detok.pop(req.request_id, None)
        return outs

    def _make_output(self, req: Request) -> RequestOutput:
        new = req.output_token_ids[req.num_emitted_tokens:]
        req.num_emitted_tokens = len(req.output_token_ids)
        det = self._detok.get(req.request_id)
        if det is not None:
            det.add(new)
            text = det.text
        else:
            text = ""
        fin = req.is_finished()
        comp = CompletionOutput(index=0, text=text, token_ids=list(req.output_token_ids),
                                finish_reason=FINISH_REASON.get(req.status) if fin else None,
                                stop_reason=req.stop_reason)
        stream_keys = getattr(self.model, "stream_output_keys", ())
        if not fin and not self.generation and stream_keys and (
                self.stream_mm_interval <= 1 or len(req.output_token_ids) % self.stream_mm_interval == 0):
            # streaming: only what is new since the last report (e.g. codec frames for the vocoder)
            sent = req.runtime_state.setdefault("_mm_sent", {})
            mm = {}
            for k in stream_keys:
                parts = req.multimodal_outputs.get(k) or []
                new_parts = parts[sent.get(k, 0):]
                sent[k] = len(parts)
                if new_parts:
                    mm[k] = torch.cat(new_parts, dim=0)
            comp.multimodal_output = mm
        if fin or self.generation:
            mm = {}
            for k, parts in req.multimodal_outputs.items():
                ts = [p for p in parts if isinstance(p, torch.Tensor)]
                mm[k] = torch.cat(ts, dim=0) if ts and len(ts) == len(parts) and ts[0].dim() > 0 else (
                    parts[0] if len(parts) == 1 else parts)
            comp.multimodal_output = mm
        metrics = {"arrival_time": req.arrival_time, "first_token_time": req.first_token_time,
                   "num_prompt_tokens": req.num_prompt_tokens, "num_output_tokens": len(req.output_token_ids)}
        return RequestOutput(request_id=req.request_id, prompt=req.prompt, prompt_token_ids=req.prompt_token_ids,
                             outputs=[comp], finished=fin, metrics=metrics,
                             multimodal_output=comp.multimodal_output)

    def update_request(self, request_id: str, payload: dict) -> bool:
        """Late input for a running request (rows of an upstream stage that is still generating): handed to the
        model's ``on_stream_update``.  Unknown or finished requests are ignored."""
        req = self._reqs.get(request_id)
        fn = getattr(self.model, "on_stream_update", None)
        if req is None or fn is None or req.is_finished():
            return False
        fn(req, payload)
        return True

    def generate(self, prompts, sampling_params=None) -> list[RequestOutput]:
        """Blocking convenience wrapper: run the given prompts to completion."""
        if isinstance(prompts, (str, dict)):
            prompts = [prompts]
        sps = sampling_params if isinstance(sampling_params, (list, tuple)) else [sampling_params] * len(prompts)
        ids = [f"gen-{i}-{time.monotonic_ns()}" for i in range(len(prompts))]
        for rid, p, sp in zip(ids, prompts, sps):
            self.add_request(rid, p, sp)
        final: dict[str, RequestOutput] = {}
        while len(final) < len(ids):
            for o in self.step():
                if o.finished and o.request_id in ids:
                    final[o.request_id] = o
            if not self.has_unfinished_requests() and len(final) < len(ids):
                raise RuntimeError("engine drained before all requests finished")
        return [final[r] for r in ids]
