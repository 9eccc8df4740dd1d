from .allocator import AllocatorError, PageAllocator  # noqa: F401
from .manager import CacheManager, CacheError, SeqCache  # noqa: F401
