"""Prompt and sampling-parameter types of the public API.

Field names follow the reference (vllm_omni/inputs/data.py:20-284) so user scripts port
unchanged; ``SamplingParams`` is this framework's own AR sampling configuration (the
reference borrows vLLM's).
"""
from __future__ import annotations

import copy
import pprint
from dataclasses import asdict, dataclass, field
from typing import Any, TypedDict, Union

import torch

try:  # Python 3.11+
    from typing import NotRequired
except ImportError:  # pragma: no cover
    from typing_extensions import NotRequired


class OmniTextPrompt(TypedDict):
    prompt: str
    negative_prompt: NotRequired[str]
    multi_modal_data: NotRequired[dict[str, Any]]
    mm_processor_kwargs: NotRequired[dict[str, Any]]
    prompt_embeds: NotRequired[torch.Tensor]
    negative_prompt_embeds: NotRequired[torch.Tensor]
    additional_information: NotRequired[dict[str, Any]]


class OmniTokensPrompt(TypedDict):
    prompt_token_ids: list[int]
    prompt: NotRequired[str]
    multi_modal_data: NotRequired[dict[str, Any]]
    prompt_embeds: NotRequired[torch.Tensor]
    additional_information: NotRequired[dict[str, Any]]
    cache_salt: NotRequired[str]


class OmniEmbedsPrompt(TypedDict):
    prompt_embeds: torch.Tensor
    prompt_embeds_mask: NotRequired[torch.Tensor]
    negative_prompt_embeds: NotRequired[torch.Tensor]
    negative_prompt_embeds_mask: NotRequired[torch.Tensor]
    additional_information: NotRequired[dict[str, Any]]
    cache_salt: NotRequired[str]


OmniPromptType = Union[str, OmniTextPrompt, OmniTokensPrompt, OmniEmbedsPrompt]


def token_inputs_omni(prompt_token_ids, prompt=None, cache_salt=None, prompt_embeds=None,
                      additional_information=None) -> dict:
    inputs: dict[str, Any] = {"type": "token", "prompt_token_ids": list(prompt_token_ids)}
    if prompt is not None:
        inputs["prompt"] = prompt
    if cache_salt is not None:
        inputs["cache_salt"] = cache_salt
    if prompt_embeds is not None:
        inputs["prompt_embeds"] = prompt_embeds
    if additional_information is not None:
        inputs["additional_information"] = additional_information
    return inputs


@dataclass
class SamplingParams:
    """AR sampling configuration (temperature / top-k / top-p / penalties / stop)."""
    n: int = 1
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0                      # 0 or -1 = disabled
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    seed: int | None = None
    max_tokens: int | None = 16
    min_tokens: int = 0
    stop: list[str] | None = None
    stop_token_ids: list[int] | None = None
    ignore_eos: bool = False
    logprobs: int | None = None
    detokenize: bool = True
    skip_special_tokens: bool = True
    suppress_token_ids: list[int] | None = None   # talker-style logits masking
    extra_args: dict[str, Any] = field(default_factory=dict)

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if not 0 < self.top_p <= 1:
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k is None or self.top_k < 0:
            self.top_k = 0
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be > 0")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0

    def clone(self) -> "SamplingParams":
        return copy.deepcopy(self)


@dataclass
class LoRARequest:
    """Adapter reference: name, stable integer id and a PEFT directory."""
    lora_name: str
    lora_int_id: int
    lora_path: str = ""
    scale: float = 1.0


@dataclass
class OmniDiffusionSamplingParams:
    """Everything a diffusion pipeline needs for one request."""
    max_sequence_length: int | None = None
    prompt_template: dict[str, Any] | None = None
    do_classifier_free_guidance: bool = False
    num_outputs_per_prompt: int = 1
    seed: int | None = None
    generator: Any = None
    generator_device: str | None = None
    layers: int = 4
    cfg_normalize: bool = False
    use_en_prompt: bool = False
    resolution: int = 640
    is_prompt_processed: bool = False
    latents: torch.Tensor | None = None
    raw_latent_shape: Any = None
    noise_pred: torch.Tensor | None = None
    image_latent: torch.Tensor | None = None
    height_latents: Any = None
    width_latents: Any = None
    num_frames: int = 1
    num_frames_round_down: bool = False
    height: int | None = None
    width: int | None = None
    fps: int | None = None
    height_not_provided: bool = False
    width_not_provided: bool = False
    timesteps: torch.Tensor | None = None
    timestep: Any = None
    step_index: int | None = None
    boundary_ratio: float | None = None
    num_inference_steps: int = 50
    guidance_scale: float = 0.0
    guidance_scale_provided: bool = False
    guidance_scale_2: float | None = None
    guidance_rescale: float = 0.0
    eta: float = 0.0
    sigmas: list[float] | None = None
    true_cfg_scale: float | None = None
    n_tokens: int | None = None
    extra_step_kwargs: dict[str, Any] = field(default_factory=dict)
    past_key_values: Any = None
    kv_metadata: dict[str, Any] | None = None
    need_kv_receive: bool = True
    modules: dict[str, Any] = field(default_factory=dict)
    return_trajectory_latents: bool = False
    return_trajectory_decoded: bool = False
    trajectory_timesteps: Any = None
    trajectory_latents: torch.Tensor | None = None
    extra_args: dict[str, Any] = field(default_factory=dict)
    save_output: bool = True
    return_frames: bool = False
    output_type: str = "pil"
    lora_request: LoRARequest | None = None
    lora_scale: float = 1.0
    profile: bool = False
    num_profiled_timesteps: int = 8
    debug: bool = False
    output: torch.Tensor | None = None

    @property
    def batch_size(self) -> int:
        return self.num_outputs_per_prompt

    def __str__(self):
        d = {k: v for k, v in asdict(self).items() if not isinstance(v, torch.Tensor)}
        return pprint.pformat(d, indent=2, width=120)

    def clone(self) -> "OmniDiffusionSamplingParams":
        return copy.deepcopy(self)


OmniSamplingParams = Union[SamplingParams, OmniDiffusionSamplingParams]
