from .manager import (
    CacheError,
    CacheGroup,
    CacheManager,
    LayerMemory,
    OutOfPages,
    PagePool,
    RequestCache,
)

__all__ = [
    "CacheError",
    "CacheGroup",
    "CacheManager",
    "LayerMemory",
    "OutOfPages",
    "PagePool",
    "RequestCache",
]
