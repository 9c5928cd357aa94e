from .data import (LoRARequest, OmniDiffusionSamplingParams, OmniEmbedsPrompt, OmniPromptType, OmniSamplingParams,
                   OmniTextPrompt, OmniTokensPrompt, SamplingParams, token_inputs_omni)

__all__ = ["LoRARequest", "OmniDiffusionSamplingParams", "OmniEmbedsPrompt", "OmniPromptType", "OmniSamplingParams",
           "OmniTextPrompt", "OmniTokensPrompt", "SamplingParams", "token_inputs_omni"]
