from .slots import SlotAllocator, SlotError
from .storage import PAGE, Cache, CacheFull, CacheNeed, CacheView

__all__ = ["SlotAllocator", "SlotError", "Cache", "CacheFull", "CacheNeed", "CacheView", "PAGE"]
