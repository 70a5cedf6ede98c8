from .paged import CACHE_KINDS, Cache, CacheStorage, CacheView
from .slots import PAGE, CacheError, FreeList, SequenceTable
