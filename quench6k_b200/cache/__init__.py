from .manager import CacheManager, GroupSpec, OutOfPages, OutOfSlots, PagePool, SlotPool
