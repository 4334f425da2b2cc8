from .allocator import OutOfPages, PageAllocator
from .manager import CacheManager, KVGroup, KVNeed, StateSlots

__all__ = ["OutOfPages", "PageAllocator", "CacheManager", "KVGroup", "KVNeed", "StateSlots"]
