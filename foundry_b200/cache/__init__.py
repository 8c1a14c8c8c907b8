"""The cache: slots and pages on the host, grouped storage on the device."""
from .pages import PAGE, CacheError, CacheFull, CacheMisuse, FreeList, GroupPages, SlotTable, pages_for
from .store import KVGroup, KVRequest, KVView, SequenceCache, StateRequest, StateView

__all__ = ["PAGE", "CacheError", "CacheFull", "CacheMisuse", "FreeList", "GroupPages", "SlotTable",
           "pages_for", "KVGroup", "KVRequest", "KVView", "SequenceCache", "StateRequest",
           "StateView"]
