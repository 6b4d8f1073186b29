from .cache import PAGE_TOKENS, Cache, CacheHandle, KVEntryView, KVRequest, Request, StateRequest
from .pages import CacheFull, CacheMisuse, PagePool, SlotTable

__all__ = ["PAGE_TOKENS", "Cache", "CacheHandle", "KVEntryView", "KVRequest", "Request", "StateRequest",
           "CacheFull", "CacheMisuse", "PagePool", "SlotTable"]
