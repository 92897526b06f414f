from .manager import CacheError, CacheGroup, CacheManager, PagePool, groups_for  # noqa: F401
