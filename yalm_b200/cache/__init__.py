from .slots import SlotAllocator, SlotError
from .storage import Cache, CacheNeed, CacheView

__all__ = ["SlotAllocator", "SlotError", "Cache", "CacheNeed", "CacheView"]
