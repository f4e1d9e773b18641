"""The cache: pages of keys and values per group of layers, fixed-size state per sequence slot."""
from .allocator import CacheBook, CacheFull, CacheMisuse, IndexPool, Sequence_
from .paged import PagedCache, PAGE_SIZE
