"""axono.nn, the KV-cache part (axono/python/axono/nn/kv_cache.py:41-117)."""
from .kv_cache import DynamicKVCache, KVCache, PagedKVCache  # noqa: F401
