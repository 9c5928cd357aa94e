from .model import build_qwen3_tts_stage  # noqa: F401
