from .paged import PagedKVCache, compute_block_hash
from .protocol import KVCacheManager
from .radix import RadixKVCache

__all__ = ["PagedKVCache", "RadixKVCache", "KVCacheManager", "compute_block_hash"]
