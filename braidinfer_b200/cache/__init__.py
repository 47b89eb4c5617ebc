"""The cache: pages of keys and values per layer group, slots per sequence, fixed-size state."""
from .pages import CacheError, GroupPages, PagePool, SlotTable
from .manager import PAGE_SIZE, CacheGroup, CacheManager, LayerCache
