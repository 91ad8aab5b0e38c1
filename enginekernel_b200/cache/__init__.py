"""The cache: sequence slots, paged keys and values per layer group, fixed-size state."""
from .pages import PAGE, CacheError, FreeList, PageGroup, SlotBook
from .store import EntryView, SequenceCache

__all__ = ["PAGE", "CacheError", "FreeList", "PageGroup", "SlotBook", "EntryView", "SequenceCache"]
