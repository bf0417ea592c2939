from .manager import PAGE_SIZE, CacheManager, FixedState, NoSlot, PagedGroup, PagedKV, Request, StateGroup
from .pages import PagePool, PoolFull

__all__ = ["PAGE_SIZE", "CacheManager", "FixedState", "NoSlot", "PagedGroup", "PagedKV", "Request", "StateGroup",
           "PagePool", "PoolFull"]
