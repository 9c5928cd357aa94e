from .manager import DiffusionLoRAManager  # noqa: F401
