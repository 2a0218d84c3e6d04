from .manager import (
    NO_PAGE,
    CacheCapacityFull,
    CacheManager,
    DoubleFreeError,
    GroupSpec,
    PageAllocator,
)

__all__ = [
    "NO_PAGE", "CacheCapacityFull", "CacheManager", "DoubleFreeError", "GroupSpec", "PageAllocator",
]
