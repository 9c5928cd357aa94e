"""Entry-point plugins (vllm_omni/plugins/__init__.py): packages may register extra pipelines,
AR models or connectors by exposing a callable in the ``vllm_omni_b200.general_plugins`` entry
point group (the reference's group names are honoured too)."""
from __future__ import annotations

import importlib.metadata as md
import os

from ..logger import init_logger

logger = init_logger(__name__)
GROUPS = ("vllm_omni_b200.general_plugins", "vllm_omni.general_plugins")
_loaded = False


def load_plugins_by_group(group: str) -> dict:
    allowed = os.environ.get("OMNI_PLUGINS")
    allowed = set(allowed.split(",")) if allowed else None
    found = {}
    try:
        eps = md.entry_points(group=group)
    except TypeError:      # pragma: no cover
        eps = md.entry_points().get(group, [])
    for ep in eps:
        if allowed is not None and ep.name not in allowed:
            continue
        try:
            found[ep.name] = ep.load()
        except Exception:   # noqa: BLE001
            logger.exception("plugin %s failed to load", ep.name)
    return found


def load_general_plugins() -> None:
    global _loaded
    if _loaded:
        return
    _loaded = True
    for g in GROUPS:
        for name, fn in load_plugins_by_group(g).items():
            try:
                fn()
            except Exception:   # noqa: BLE001
                logger.exception("plugin %s raised during registration", name)
