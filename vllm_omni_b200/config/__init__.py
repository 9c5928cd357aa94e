"""Configuration entry points gathered in one place (vllm_omni/config/model.py and the
dataclasses of vllm_omni/diffusion/data.py, vllm_omni/engine/arg_utils.py)."""
from ..diffusion.data import (DiffusionCacheConfig, DiffusionParallelConfig, OmniDiffusionConfig,  # noqa: F401
                              TransformerConfig)
from ..entrypoints.omni_llm import OmniEngineArgs  # noqa: F401
from ..entrypoints.utils import OmniPipelineConfig, StageConfig, load_stage_configs_from_yaml  # noqa: F401
from ..models.qwen_decoder import DecoderConfig as OmniModelConfig  # noqa: F401
