from .model import build_qwen2_5_omni_stage  # noqa: F401
