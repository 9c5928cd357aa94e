"""vllm_omni_b200 — Blackwell-native omni-modality serving.

Public API (same names as the reference package): ``Omni``, ``AsyncOmni``,
``OmniDiffusionSamplingParams``, ``SamplingParams``, ``OmniRequestOutput``.
"""
__version__ = "0.1.0"


def __getattr__(name):
    if name == "Omni":
        from .entrypoints.omni import Omni
        return Omni
    if name == "AsyncOmni":
        from .entrypoints.async_omni import AsyncOmni
        return AsyncOmni
    if name in ("OmniDiffusionSamplingParams", "SamplingParams", "OmniTextPrompt", "OmniTokensPrompt",
                "OmniEmbedsPrompt", "LoRARequest"):
        from . import inputs
        return getattr(inputs, name)
    if name in ("OmniRequestOutput", "RequestOutput", "CompletionOutput"):
        from . import outputs
        return getattr(outputs, name)
    raise AttributeError(name)


__all__ = ["Omni", "AsyncOmni", "OmniDiffusionSamplingParams", "SamplingParams", "OmniRequestOutput", "__version__"]
