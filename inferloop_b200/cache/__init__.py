from .manager import CacheManager, LayerCache, PageGroup
from .pages import OutOfPages, PageLedgerError, PagePool
from .slots import OutOfSlots, SlotPool

__all__ = ["CacheManager", "LayerCache", "PageGroup", "OutOfPages", "PageLedgerError",
           "PagePool", "OutOfSlots", "SlotPool"]
