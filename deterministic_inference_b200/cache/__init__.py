from .manager import CacheError, CacheManager, CacheView, OutOfPages, PageGroup
