from astrai_b200.inference.cache.buffer import KVCache, KVStorage, ReqToTokenPool
from astrai_b200.inference.cache.pool import DEFAULT_PAGE_SIZE, PagePool, TaskCacheManager, page_hash
from astrai_b200.inference.cache.strategy import (
    AllocationStrategy, Allocator, ContiguousStrategy, PagedStrategy, RadixCache, TaskCacheState,
)

__all__ = [
    "AllocationStrategy", "Allocator", "ContiguousStrategy", "DEFAULT_PAGE_SIZE", "KVCache", "KVStorage", "PagePool",
    "PagedStrategy", "RadixCache", "ReqToTokenPool", "TaskCacheManager", "TaskCacheState", "page_hash",
]
