from .native import CacheError
from .allocator import BlockAllocator
from .manager import CacheManager, OutOfPages

__all__ = ["CacheError", "BlockAllocator", "CacheManager", "OutOfPages"]
