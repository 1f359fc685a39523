from .allocator import BlockAllocator, OutOfBlocks, OutOfPages
from .manager import BlockTable, CacheManager, CacheView, PagedGroup, SequenceCache, StateGroup

__all__ = ["BlockAllocator", "OutOfBlocks", "OutOfPages", "BlockTable", "CacheManager", "CacheView",
           "PagedGroup", "SequenceCache", "StateGroup"]
