from .block_allocator import BlockAllocator, PageError
from .manager import SCRATCH_PAGE, CacheManager, KVGroup, OutOfPages, RequestCache, plan_groups
from .spec import PagedKVSpec, StateSpec

__all__ = ["BlockAllocator", "PageError", "CacheManager", "KVGroup", "OutOfPages", "RequestCache",
           "PagedKVSpec", "StateSpec", "SCRATCH_PAGE", "plan_groups"]
