from .block_pool import BlockPool, PagePoolError
from .manager import CacheManager, NoCapacity, page_hashes
from .storage import CacheStorage, page_bytes

__all__ = ["BlockPool", "PagePoolError", "CacheManager", "NoCapacity", "page_hashes", "CacheStorage",
           "page_bytes"]
