"""Result types returned by ``Omni`` / ``AsyncOmni``.

``OmniRequestOutput`` keeps the reference's two-mode shape (vllm_omni/outputs.py:29-253):
pipeline-stage outputs wrap a ``RequestOutput`` (text tokens plus multimodal tensors) and
diffusion outputs carry images / latents directly.  ``RequestOutput`` and
``CompletionOutput`` are this framework's own AR result records (the reference borrows
vLLM's).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch


@dataclass
class CompletionOutput:
    index: int = 0
    text: str = ""
    token_ids: list[int] = field(default_factory=list)
    cumulative_logprob: float | None = None
    logprobs: Any = None
    finish_reason: str | None = None
    stop_reason: Any = None
    multimodal_output: dict[str, Any] = field(default_factory=dict)

    def finished(self) -> bool:
        return self.finish_reason is not None


@dataclass
class RequestOutput:
    request_id: str = ""
    prompt: str | None = None
    prompt_token_ids: list[int] | None = None
    outputs: list[CompletionOutput] = field(default_factory=list)
    finished: bool = False
    metrics: dict[str, Any] = field(default_factory=dict)
    multimodal_output: dict[str, Any] = field(default_factory=dict)
    num_cached_tokens: int | None = None
    encoder_prompt_token_ids: list[int] | None = None
    prompt_logprobs: Any = None
    kv_transfer_params: Any = None


@dataclass
class OmniModelRunnerOutput:
    """What a model runner hands back to its scheduler after one step."""
    req_ids: list[str] = field(default_factory=list)
    sampled_token_ids: list[list[int]] = field(default_factory=list)
    multimodal_outputs: dict[str, Any] | None = None
    pooler_output: list[Any] | None = None
    # requests whose KV pages were handed to the connector; the scheduler may free them
    kv_extracted_req_ids: list[str] | None = None


@dataclass
class OmniRequestOutput:
    request_id: str = ""
    finished: bool = True
    stage_id: int | None = None
    final_output_type: str = "text"
    request_output: RequestOutput | None = None
    images: list[Any] = field(default_factory=list)
    prompt: Any = None
    latents: torch.Tensor | None = None
    metrics: dict[str, Any] = field(default_factory=dict)
    _multimodal_output: dict[str, Any] = field(default_factory=dict)
    error: str | None = None

    @classmethod
    def from_pipeline(cls, stage_id: int, final_output_type: str, request_output: RequestOutput):
        return cls(request_id=getattr(request_output, "request_id", ""), stage_id=stage_id,
                   final_output_type=final_output_type, request_output=request_output,
                   finished=getattr(request_output, "finished", True))

    @classmethod
    def from_diffusion(cls, request_id: str, images: list, prompt=None, metrics=None, latents=None,
                       multimodal_output=None, final_output_type: str = "image"):
        return cls(request_id=request_id, final_output_type=final_output_type, images=images, prompt=prompt,
                   latents=latents, metrics=metrics or {}, _multimodal_output=multimodal_output or {}, finished=True)

    @property
    def multimodal_output(self) -> dict[str, Any]:
        if self.request_output is not None:
            for o in getattr(self.request_output, "outputs", None) or []:
                mm = getattr(o, "multimodal_output", None)
                if mm:
                    return mm
            return getattr(self.request_output, "multimodal_output", {}) or {}
        return self._multimodal_output

    @property
    def num_images(self) -> int:
        return len(self.images)

    @property
    def prompt_token_ids(self):
        return getattr(self.request_output, "prompt_token_ids", None)

    @property
    def outputs(self) -> list:
        return getattr(self.request_output, "outputs", []) if self.request_output is not None else []

    @property
    def encoder_prompt_token_ids(self):
        return getattr(self.request_output, "encoder_prompt_token_ids", None)

    @property
    def prompt_logprobs(self):
        return getattr(self.request_output, "prompt_logprobs", None)

    @property
    def num_cached_tokens(self):
        return getattr(self.request_output, "num_cached_tokens", None)

    @property
    def kv_transfer_params(self):
        return getattr(self.request_output, "kv_transfer_params", None)

    @property
    def is_diffusion_output(self) -> bool:
        return self.request_output is None

    @property
    def is_pipeline_output(self) -> bool:
        return self.request_output is not None

    def to_dict(self) -> dict[str, Any]:
        d = {"request_id": self.request_id, "finished": self.finished, "final_output_type": self.final_output_type,
             "stage_id": self.stage_id, "metrics": self.metrics}
        if self.is_diffusion_output:
            d.update(num_images=self.num_images, prompt=self.prompt if isinstance(self.prompt, str) else None)
        else:
            d.update(text=[o.text for o in self.outputs])
        return d

    def __repr__(self) -> str:
        if self.is_diffusion_output:
            return (f"OmniRequestOutput(request_id={self.request_id!r}, type={self.final_output_type}, "
                    f"images={self.num_images}, finished={self.finished})")
        return (f"OmniRequestOutput(request_id={self.request_id!r}, stage={self.stage_id}, "
                f"type={self.final_output_type}, finished={self.finished})")
