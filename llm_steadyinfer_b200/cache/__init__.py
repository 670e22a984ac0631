from .manager import CacheGroup, CacheLayout, CacheManager, OutOfPages, OutOfSlots
from .pages import PageError, PagePool, SlotPool
from .storage import CacheStorage, LayerCache
