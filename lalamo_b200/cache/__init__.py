"""The cache manager: pages, block tables, state slots."""

from .manager import CacheLayout, CacheManager, RequestCache, plan_cache_layout
from .pages import OutOfPages, OutOfSlots, PagePool, SlotPool

__all__ = [
    "CacheLayout",
    "CacheManager",
    "OutOfPages",
    "OutOfSlots",
    "PagePool",
    "RequestCache",
    "SlotPool",
    "plan_cache_layout",
]
