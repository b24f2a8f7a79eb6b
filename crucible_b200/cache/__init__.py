from .pages import CacheError, PagePool, PoolExhausted, StateSlotPool
from .manager import RELEASED, CacheManager, GroupPolicy
