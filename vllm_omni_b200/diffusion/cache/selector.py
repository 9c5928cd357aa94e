"""Cache backend selection by name (``cache_backend`` engine argument or the
``DIFFUSION_CACHE_BACKEND`` environment variable, vllm_omni/diffusion/cache/selector.py)."""
from __future__ import annotations

from .base import CacheBackend


def get_cache_backend(name: str | None, config) -> CacheBackend | None:
    n = (name or "none").lower().replace("-", "_")
    if n in ("none", ""):
        return None
    if n in ("tea_cache", "teacache"):
        from .teacache import TeaCacheBackend
        return TeaCacheBackend(config)
    if n in ("cache_dit", "dbcache", "db_cache"):
        from .dbcache import DBCacheBackend
        return DBCacheBackend(config)
    raise ValueError(f"unknown cache backend {name!r}: expected none, tea_cache or cache_dit")
