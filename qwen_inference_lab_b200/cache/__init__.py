from .manager import CacheError, CacheManager, KVCacheView, OutOfPages, StateView
