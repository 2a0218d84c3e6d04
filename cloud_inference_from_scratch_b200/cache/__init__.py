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


def __getattr__(name):  # the device side needs torch; the host side must import without it
    if name in ("CachePools", "plan_groups", "pages_from_bytes"):
        from . import pools

        return getattr(pools, name)
    raise AttributeError(name)
