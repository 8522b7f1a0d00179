from matricxon_b200.cache.manager import (
    CacheError,
    CacheManager,
    GroupRule,
    OutOfPages,
    PagePool,
    RequestRecord,
    SlotPool,
)

__all__ = ["CacheError", "CacheManager", "GroupRule", "OutOfPages", "PagePool", "RequestRecord",
           "SlotPool"]
