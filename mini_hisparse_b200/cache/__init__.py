from .allocator import CapacityError, PageAllocator
from .manager import CacheConfig, CacheManager, PageGroup, StateGroup
