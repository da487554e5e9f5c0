"""Cache manager: pages with block tables per request and per group, and slots for state of fixed size."""
from .pages import CacheError, PagePool, page_hash
from .manager import CacheManager, PagedKV, SlotState, PageGroup

__all__ = ["CacheError", "PagePool", "page_hash", "CacheManager", "PagedKV", "SlotState", "PageGroup"]
