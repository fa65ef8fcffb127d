from .manager import PagedCache, CacheConfig
