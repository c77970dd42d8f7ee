from .manager import CacheManager, RequestCache
from .page_pool import OutOfPages, PagePool, PagePoolError
from .slots import NoFreeSlot, SlotPool
from .storage import CacheStorage, GroupLayout, plan_groups
