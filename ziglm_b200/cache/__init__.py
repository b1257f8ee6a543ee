from .slots import (CacheError, CacheFull, FreeList, GroupPages, NoFreeSlot, SequenceTooLong, SlotTable)
from .storage import PAGE_SIZE, CacheStorage, KVGroup

__all__ = ["CacheError", "CacheFull", "FreeList", "GroupPages", "NoFreeSlot", "SequenceTooLong", "SlotTable",
           "PAGE_SIZE", "CacheStorage", "KVGroup"]
