"""Per-sequence storage: pages of keys and values, fixed-size records, and the slots that own them."""

from .cache import PAGE_SIZE, Cache, KVGroup, KVView, PagePool, StateGroup, StateView

__all__ = ["PAGE_SIZE", "Cache", "KVGroup", "KVView", "PagePool", "StateGroup", "StateView"]
