"""The cache: slots, pages, per-sequence lengths, fixed-size per-sequence state."""
from .allocators import CacheError, CacheFull, ContextLengthExceeded, IdAllocator
from .cache import Cache, CacheView

__all__ = ["CacheError", "CacheFull", "ContextLengthExceeded", "IdAllocator", "Cache", "CacheView"]
