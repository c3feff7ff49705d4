"""Cache manager: pages of keys and values per group of layers, a block table
per request, and slots for per-request state of fixed size."""

from gllm_b200.cache.allocator import BlockAllocator, CacheError, OutOfPages, SlotAllocator
from gllm_b200.cache.manager import CacheGroup, CacheManager, RequestCache

__all__ = [
    "BlockAllocator", "CacheError", "OutOfPages", "SlotAllocator",
    "CacheGroup", "CacheManager", "RequestCache",
]
