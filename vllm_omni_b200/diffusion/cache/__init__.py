from .base import CacheBackend  # noqa: F401
from .selector import get_cache_backend  # noqa: F401
