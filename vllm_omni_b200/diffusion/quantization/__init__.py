from .fp8 import DiffusionFp8Config, fp8_linear, quantize_pipeline, quantize_weight_blockwise  # noqa: F401
