from .paged import Cache, CacheView
from .slots import PAGE, CacheError, FreeList, SequenceTable
