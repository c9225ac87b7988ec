from .allocator import DoubleFree, IdAllocator
from .manager import CacheGroup, CacheManager, pages_for

__all__ = ["CacheGroup", "CacheManager", "DoubleFree", "IdAllocator", "pages_for"]
