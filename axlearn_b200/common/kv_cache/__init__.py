"""KV caches for incremental decoding: dense, sliding-window ring buffer, and paged."""

from axlearn_b200.common.kv_cache.base_kv_cache import BaseKVCache, KVState  # noqa: F401
from axlearn_b200.common.kv_cache.kv_cache import KVCache  # noqa: F401
from axlearn_b200.common.kv_cache.paged_kv_cache import PagedKVCache  # noqa: F401
from axlearn_b200.common.kv_cache.sliding_window_kv_cache import SlidingWindowKVCache  # noqa: F401
