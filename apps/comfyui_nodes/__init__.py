"""ComfyUI custom nodes that talk to a running server over HTTP (the role of the reference's
``apps/ComfyUI-vLLM-Omni``).  Drop this folder into ``ComfyUI/custom_nodes``."""
from .nodes import NODE_CLASS_MAPPINGS, NODE_DISPLAY_NAME_MAPPINGS  # noqa: F401
