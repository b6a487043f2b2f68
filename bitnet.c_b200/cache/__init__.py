"""The cache: slots, paged keys and values per group of runs, fixed-size per-sequence state."""
from .pages import PAGE, CacheError, CacheFull, PagePool, SlotTable, pages_for
from .cache import Cache, KvGroup, KvView

__all__ = ["PAGE", "CacheError", "CacheFull", "PagePool", "SlotTable", "pages_for", "Cache", "KvGroup", "KvView"]
