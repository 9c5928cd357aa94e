"""Request state of the AR engine (the roles of vllm_omni/request.py ``OmniRequest`` and
vllm_omni/engine/__init__.py ``OmniEngineCoreRequest``): prompt tokens or prompt embeddings,
per-request ``additional_information`` tensors for the model's preprocess hook, sampling
parameters, paged-KV block table and the extra ``WAITING_FOR_CHUNK`` status used when a
stage consumes its input as a stream of chunks from the previous stage."""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import Any

import torch

from ..inputs.data import SamplingParams


class RequestStatus(enum.IntEnum):
    WAITING_FOR_CHUNK = -1
    WAITING = 0
    RUNNING = 1
    PREEMPTED = 2
    FINISHED_STOPPED = 3
    FINISHED_LENGTH = 4
    FINISHED_ABORTED = 5
    FINISHED_ERROR = 6

    @property
    def finished(self) -> bool:
        return self >= RequestStatus.FINISHED_STOPPED


FINISH_REASON = {RequestStatus.FINISHED_STOPPED: "stop", RequestStatus.FINISHED_LENGTH: "length",
                 RequestStatus.FINISHED_ABORTED: "abort", RequestStatus.FINISHED_ERROR: "error"}


@dataclass(eq=False)          # identity semantics: queues look requests up by object, never by field values
class Request:
    request_id: str
    prompt_token_ids: list[int]
    sampling_params: SamplingParams
    prompt: str | None = None
    prompt_embeds: torch.Tensor | None = None              # [len(prompt), hidden] overlay for token embeddings
    additional_information: dict[str, Any] = field(default_factory=dict)
    multi_modal_data: dict[str, Any] | None = None
    eos_token_id: int | None = None
    arrival_time: float = field(default_factory=time.time)
    status: RequestStatus = RequestStatus.WAITING
    output_token_ids: list[int] = field(default_factory=list)
    num_computed_tokens: int = 0                           # tokens whose KV is in the cache
    block_ids: list[int] = field(default_factory=list)
    num_emitted_tokens: int = 0                            # output tokens already reported (streaming)
    multimodal_outputs: dict[str, list] = field(default_factory=dict)
    first_token_time: float | None = None
    # streaming input (async chunk): more prompt chunks may arrive while the request runs
    expects_more_chunks: bool = False
    chunks_received: int = 0
    # KV hand-off to another stage
    kv_transfer_requested: bool = False
    kv_transfer_done: bool = False
    stop_reason: Any = None
    decode_blocked: bool = False       # the model cannot build this request's next input yet (it waits for a stream update)
    runtime_state: dict[str, Any] = field(default_factory=dict)   # per-request model scratch (e.g. talker codes)

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    @property
    def all_token_ids(self) -> list[int]:
        return self.prompt_token_ids + self.output_token_ids

    def token_slice(self, start: int, n: int) -> list[int]:
        """``all_token_ids[start:start + n]`` without building the concatenated list (the decode step asks
        for one token of every running request)."""
        P = len(self.prompt_token_ids)
        if start >= P:
            return self.output_token_ids[start - P:start - P + n]
        if start + n <= P:
            return self.prompt_token_ids[start:start + n]
        return self.prompt_token_ids[start:] + self.output_token_ids[:start + n - P]

    @property
    def max_tokens(self) -> int:
        return self.sampling_params.max_tokens if self.sampling_params.max_tokens is not None else 1 << 30

    def append_prompt_chunk(self, token_ids: list[int], embeds: torch.Tensor | None = None, last: bool = False):
        self.prompt_token_ids = self.prompt_token_ids + list(token_ids)
        if embeds is not None:
            self.prompt_embeds = embeds if self.prompt_embeds is None else torch.cat([self.prompt_embeds, embeds], 0)
        self.chunks_received += 1
        self.expects_more_chunks = not last
        if self.status == RequestStatus.WAITING_FOR_CHUNK:
            self.status = RequestStatus.WAITING

    def is_finished(self) -> bool:
        return self.status.finished
