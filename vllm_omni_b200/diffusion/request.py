"""Request object handed from the engine to the pipelines
(vllm_omni/diffusion/request.py:10-46)."""
from __future__ import annotations

from dataclasses import dataclass, field

from ..inputs.data import OmniDiffusionSamplingParams, OmniPromptType


@dataclass
class OmniDiffusionRequest:
    prompts: list[OmniPromptType]
    sampling_params: OmniDiffusionSamplingParams
    request_ids: list[str] = field(default_factory=list)

    def __post_init__(self):
        sp = self.sampling_params
        if sp.guidance_scale > 1.0 and any((not isinstance(p, str) and p.get("negative_prompt")) for p in self.prompts):
            sp.do_classifier_free_guidance = True
        if sp.guidance_scale_2 is None:
            sp.guidance_scale_2 = sp.guidance_scale
        if sp.guidance_scale:
            sp.guidance_scale_provided = True
        else:
            sp.guidance_scale = 1.0
