from .pools import PagePool, SlotPool
from .manager import CacheManager, CacheView
