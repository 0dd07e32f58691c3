"""The cache manager: pages, block tables, groups, state slots."""
from .pages import BlockTable, CacheExhausted, PagePool, RELEASED
from .manager import CacheGroup, CacheManager, KVSpec, RequestCache, StateSlots, StateSpec

__all__ = ["BlockTable", "CacheExhausted", "PagePool", "RELEASED", "CacheGroup", "CacheManager", "KVSpec",
           "RequestCache", "StateSlots", "StateSpec"]
