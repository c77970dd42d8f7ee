from .errors import NoFreeSlot, OutOfPages, PagePoolError
from .native import NativeCacheManager
from .storage import CacheStorage, GroupLayout, plan_groups
