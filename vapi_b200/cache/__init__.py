"""Cache manager: pages for keys and values, slots for per-request state."""
from .pool import OutOfPages, OutOfSlots, PagePool, SlotPool
from .manager import CacheManager, PagedGroup, RequestCache, StateGroup

__all__ = ["OutOfPages", "OutOfSlots", "PagePool", "SlotPool", "CacheManager", "PagedGroup",
           "RequestCache", "StateGroup"]
