from .manager import CacheError, CacheFull, CacheManager, PagedKVView, SlotStateView

__all__ = ["CacheError", "CacheFull", "CacheManager", "PagedKVView", "SlotStateView"]
