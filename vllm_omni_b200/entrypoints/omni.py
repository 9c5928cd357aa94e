"""``Omni``: the offline entry point.  (Interim single-stage form; replaced by the staged
orchestrator in ``omni_orchestrator`` once stage configs are given.)"""
from __future__ import annotations

from .omni_base import Omni, OmniBase  # noqa: F401
