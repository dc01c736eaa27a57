from .kv_cache import PAGE_SIZE, CacheGroup, KvCache, KvRequest
from .pages import CacheFull, FreeList
from .state import StateArea, StateRequest
