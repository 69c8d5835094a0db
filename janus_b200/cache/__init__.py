from .pages import PAGE_SIZE, CacheFull, PagePool
from .sequence_cache import CacheView, GroupStepView, KVGroup, SequenceCache

__all__ = ["PAGE_SIZE", "CacheFull", "PagePool", "CacheView", "GroupStepView", "KVGroup", "SequenceCache"]
