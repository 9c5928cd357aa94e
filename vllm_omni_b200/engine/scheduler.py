"""Schedulers of the AR engine.

``OmniARScheduler``: continuous batching with chunked prefill under a token budget
(``max_num_batched_tokens``) and a sequence cap (``max_num_seqs``); decodes are scheduled
first, then waiting prefills; preemption by recompute when pages run out.  On top of that, the
omni-specific behaviour of the reference scheduler (vllm_omni/core/sched/omni_ar_scheduler.py:
84-136, 473-594): requests that take their prompt as a stream of chunks from the previous
stage park in ``WAITING_FOR_CHUNK``; a KV hand-off to another stage is triggered when the
prefill finishes or a special token is sampled, and pages of such a request are only freed
once the runner reports the KV as extracted.

``OmniGenerationScheduler``: one-shot scheduling for non-autoregressive stages (code2wav,
TTS decoders): the whole input is scheduled in one step and the request finishes after it
(vllm_omni/core/sched/omni_generation_scheduler.py:33-370).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from .kv_cache_manager import KVCacheManager
from .request import Request, RequestStatus


@dataclass
class ScheduledRequest:
    request: Request
    num_new_tokens: int          # tokens to run this step (prefill chunk or 1 for decode)
    start: int                   # == request.num_computed_tokens
    is_prefill: bool
    samples: bool                # whether this step produces a token for the request


@dataclass
class SchedulerOutput:
    scheduled: list[ScheduledRequest] = field(default_factory=list)
    finished_ids: list[str] = field(default_factory=list)
    kv_transfer_ids: list[str] = field(default_factory=list)     # extract KV for these after the step
    total_tokens: int = 0

    @property
    def empty(self) -> bool:
        return not self.scheduled


class OmniARScheduler:
    def __init__(self, kv: KVCacheManager, max_num_seqs: int = 64, max_num_batched_tokens: int = 8192,
                 kv_transfer_criteria: dict | None = None, chunk_adapter=None):
        self.kv = kv
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.requests: dict[str, Request] = {}
        self.kv_transfer_criteria = kv_transfer_criteria or {}
        self.chunk_adapter = chunk_adapter
        self.waiting_for_kv_extract: dict[str, Request] = {}
        self.finished_since_last: list[str] = []

    # ------------------------------------------------------------------ admission
    def add_request(self, req: Request) -> None:
        self.requests[req.request_id] = req
        if req.expects_more_chunks and not req.prompt_token_ids:
            req.status = RequestStatus.WAITING_FOR_CHUNK
        self.waiting.append(req)

    def abort(self, request_ids) -> list[Request]:
        out = []
        for rid in request_ids:
            req = self.requests.get(rid)
            if req is None or req.is_finished():
                continue
            req.status = RequestStatus.FINISHED_ABORTED
            self._release(req)
            out.append(req)
        return out

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    def has_schedulable(self) -> bool:
        return any(not r.decode_blocked for r in self.running) or any(r.status == RequestStatus.WAITING for r in self.waiting)

    # ------------------------------------------------------------------ scheduling
    def _poll_chunks(self):
        if self.chunk_adapter is None:
            return
        for req in list(self.waiting) + self.running:
            if req.expects_more_chunks:
                self.chunk_adapter.poll(req)

    def schedule(self) -> SchedulerOutput:
        self._poll_chunks()
        out = SchedulerOutput()
        budget = self.max_num_batched_tokens
        # 1. running requests: decode, continue a chunked prefill, or recompute after a preemption.
        #    What a request still has to feed is every token it owns (prompt + generated) whose KV is
        #    not in the cache; a token is sampled only by the step that feeds the last of them.
        preempted: list[Request] = []
        scheduled_ids: set[str] = set()
        for req in list(self.running):
            if budget <= 0:
                break
            if req.status != RequestStatus.RUNNING:
                continue                      # preempted earlier in this very step
            if req.decode_blocked:
                continue                      # its next input depends on a stream update that has not arrived
            remaining = req.num_tokens - req.num_computed_tokens
            if remaining <= 0:
                continue                      # everything consumed; waiting for the next chunk
            n = min(remaining, budget)
            is_prefill = not (remaining == 1 and req.output_token_ids)
            samples = (n == remaining) and not req.expects_more_chunks
            while not self.kv.allocate_slots(req, n):
                victim = self._pick_victim(exclude=req, scheduled=scheduled_ids)
                if victim is None:
                    break
                self._preempt(victim)
                preempted.append(victim)
            else:
                out.scheduled.append(ScheduledRequest(req, n, req.num_computed_tokens, is_prefill, samples))
                scheduled_ids.add(req.request_id)
                budget -= n
                continue
            # no pages even after preempting every request that is not part of this step
            self._preempt(req)
            preempted.append(req)
        # 2. admit waiting requests
        while self.waiting and budget > 0 and len(self.running) < self.max_num_seqs and not preempted:
            req = self.waiting[0]
            if req.status == RequestStatus.WAITING_FOR_CHUNK:
                # leave it parked but look at the ones behind it
                self.waiting.rotate(-1)
                if all(r.status == RequestStatus.WAITING_FOR_CHUNK for r in self.waiting):
                    break
                continue
            remaining = req.num_tokens - req.num_computed_tokens
            n = min(max(remaining, 1), budget)
            if not self.kv.allocate_slots(req, n):
                break
            self.waiting.popleft()
            req.status = RequestStatus.RUNNING
            self.running.append(req)
            samples = (n >= remaining) and not req.expects_more_chunks
            out.scheduled.append(ScheduledRequest(req, n, req.num_computed_tokens, True, samples))
            budget -= n
        out.total_tokens = self.max_num_batched_tokens - budget
        out.finished_ids, self.finished_since_last = self.finished_since_last, []
        return out

    def _pick_victim(self, exclude: Request, scheduled: set[str] = frozenset()) -> Request | None:
        """Latest-admitted running request that holds pages and is not part of the current step."""
        for r in reversed(self.running):
            if r is not exclude and r.block_ids and r.request_id not in scheduled \
                    and r.status == RequestStatus.RUNNING:
                return r
        return None

    def _preempt(self, req: Request) -> None:
        """Recompute-style preemption: drop the pages, keep the tokens, back to the queue head.
        The generated tokens stay in ``output_token_ids``; on re-admission they are fed again
        together with the prompt (``num_tokens - num_computed_tokens``)."""
        self.kv.free(req)
        req.num_computed_tokens = 0
        if req in self.running:
            self.running.remove(req)
        if req not in self.waiting:
            self.waiting.appendleft(req)
        req.status = RequestStatus.WAITING

    # ------------------------------------------------------------------ after the step
    def update_from_output(self, sched: SchedulerOutput, sampled: dict[str, int],
                           kv_extracted_req_ids: list[str] | None = None) -> list[Request]:
        """Advance request state with the tokens sampled this step; returns requests that
        produced new output (finished or not)."""
        touched = []
        for s in sched.scheduled:
            req = s.request
            if req.is_finished():
                continue
            req.num_computed_tokens += s.num_new_tokens
            if s.is_prefill and req.num_computed_tokens >= req.num_prompt_tokens and not req.expects_more_chunks:
                if self.kv_transfer_criteria.get("type") == "prefill_finished" and not req.kv_transfer_requested:
                    req.kv_transfer_requested = True
                    sched.kv_transfer_ids.append(req.request_id)
            if not s.samples or req.request_id not in sampled:
                continue
            tok = int(sampled[req.request_id])
            req.output_token_ids.append(tok)
            touched.append(req)
            if (self.kv_transfer_criteria.get("type") == "special_token"
                    and tok == self.kv_transfer_criteria.get("token_id") and not req.kv_transfer_requested):
                req.kv_transfer_requested = True
                sched.kv_transfer_ids.append(req.request_id)
            self._check_stop(req, tok)
        for rid in kv_extracted_req_ids or []:
            req = self.waiting_for_kv_extract.pop(rid, None)
            if req is not None:
                req.kv_transfer_done = True
                self.kv.free(req)
                continue
            live = self.requests.get(rid)       # still running: its pages go when it finishes
            if live is not None:
                live.kv_transfer_done = True
        for req in [r for r in self.running if r.is_finished()]:
            self._release(req)
        return touched

    def _check_stop(self, req: Request, tok: int) -> None:
        sp = req.sampling_params
        n_out = len(req.output_token_ids)
        if n_out >= sp.min_tokens:
            if not sp.ignore_eos and req.eos_token_id is not None and tok == req.eos_token_id:
                req.status, req.stop_reason = RequestStatus.FINISHED_STOPPED, None
                return
            if sp.stop_token_ids and tok in sp.stop_token_ids:
                req.status, req.stop_reason = RequestStatus.FINISHED_STOPPED, tok
                return
        if n_out >= req.max_tokens:
            req.status = RequestStatus.FINISHED_LENGTH

    def _release(self, req: Request) -> None:
        if req in self.running:
            self.running.remove(req)
        if req in self.waiting:            # (a failed ``deque.remove`` formats the request, tensors included, into its error)
            self.waiting.remove(req)
        if req.kv_transfer_requested and not req.kv_transfer_done and req.status != RequestStatus.FINISHED_ABORTED:
            self.waiting_for_kv_extract[req.request_id] = req     # pages freed once the KV is extracted
        else:
            self.kv.free(req)
        self.finished_since_last.append(req.request_id)
        self.requests.pop(req.request_id, None)


class OmniGenerationScheduler(OmniARScheduler):
    """All input tokens of a request in one step; the request finishes after that step."""

    def schedule(self) -> SchedulerOutput:
        self._poll_chunks()
        out = SchedulerOutput()
        budget = self.max_num_batched_tokens
        while self.waiting and len(out.scheduled) < self.max_num_seqs:
            req = self.waiting[0]
            if req.status == RequestStatus.WAITING_FOR_CHUNK:
                self.waiting.rotate(-1)
                if all(r.status == RequestStatus.WAITING_FOR_CHUNK for r in self.waiting):
                    break
                continue
            n = max(1, req.num_prompt_tokens - req.num_computed_tokens)
            if n > budget and out.scheduled:
                break
            self.waiting.popleft()
            req.status = RequestStatus.RUNNING
            self.running.append(req)
            out.scheduled.append(ScheduledRequest(req, n, req.num_computed_tokens, True, False))
            budget -= n
        out.total_tokens = self.max_num_batched_tokens - budget
        out.finished_ids, self.finished_since_last = self.finished_since_last, []
        return out

    def update_from_output(self, sched, sampled, kv_extracted_req_ids=None):
        touched = []
        for s in sched.scheduled:
            req = s.request
            req.num_computed_tokens += s.num_new_tokens
            if req.expects_more_chunks:
                # streaming input: stay alive, wait for the next chunk
                req.status = RequestStatus.WAITING_FOR_CHUNK
                self.running.remove(req)
                self.waiting.append(req)
            else:
                req.status = RequestStatus.FINISHED_STOPPED
                self._release(req)
            touched.append(req)
        return touched
