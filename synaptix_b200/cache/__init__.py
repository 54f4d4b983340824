from .pages import PAGE_TOKENS, CacheFull, PagePool, SequenceSlots, SlotError, pages_for
from .store import Cache, CacheRequest, KVRequest, KVView, StateRequest

__all__ = ["PAGE_TOKENS", "CacheFull", "PagePool", "SequenceSlots", "SlotError", "pages_for",
           "Cache", "CacheRequest", "KVRequest", "KVView", "StateRequest"]
