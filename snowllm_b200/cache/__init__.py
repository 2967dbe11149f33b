"""Paged key/value cache with per-request block tables in groups, and fixed-size state slots."""
from .manager import CacheManager, PagedView, RequestCache, SlotView, pages_for  # noqa: F401
from .pages import PagePool, StateSlots  # noqa: F401
