"""The cache: slots and pages on the host, keys/values and per-sequence state on the device."""
from .pages import PAGE_SIZE, CacheError, PagePool, SlotTable, pages_for  # noqa: F401
from .storage import CacheBinding, KVGroup, KVRequest, SequenceCache, StateGroup, StateRequest  # noqa: F401
