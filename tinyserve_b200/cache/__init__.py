from .allocator import OutOfPagesError, PageAllocator
from .block_table import RELEASED, BlockTable
from .manager import CacheManager, OutOfSlotsError, PageGroup, RequestCache, StatePool

__all__ = ["OutOfPagesError", "PageAllocator", "RELEASED", "BlockTable", "CacheManager",
           "OutOfSlotsError", "PageGroup", "RequestCache", "StatePool"]
