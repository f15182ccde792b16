from .manager import CacheManager, GroupInfo, Sequence_
from .pages import PagePool
from .storage import CacheStorage, CacheView

__all__ = ["CacheManager", "CacheStorage", "CacheView", "GroupInfo", "PagePool", "Sequence_"]
