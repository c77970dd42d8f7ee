from .manager import CacheManager, RequestCache
from .native import NativeCacheManager
from .page_pool import OutOfPages, PagePool, PagePoolError
from .slots import NoFreeSlot, SlotPool
from .storage import CacheStorage, GroupLayout, plan_groups
