from .paged import PAGE, CacheGroup, LayerKV, PagePool, pages_for
from .sequence_cache import SequenceCache
from .slots import CacheError, SlotAllocator
