"""The cache manager: paged keys and values, block tables, state slots."""

from .manager import CacheManager, Group, RequestCache
from .pages import PageAccountingError, PagePool

__all__ = ["CacheManager", "Group", "PageAccountingError", "PagePool", "RequestCache"]
