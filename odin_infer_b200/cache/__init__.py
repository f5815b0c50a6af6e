"""The cache: page pools, groups of layers with storage of their own, slots, per-sequence state."""
from .groups import KVGroup, KVRequest, PAGE, pages_for
from .manager import CacheManager
from .pages import CacheError, PagePool

__all__ = ["CacheError", "CacheManager", "KVGroup", "KVRequest", "PAGE", "PagePool", "pages_for"]
