from .config import Qwen3OmniConfig  # noqa: F401
