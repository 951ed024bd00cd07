from .allocator import CacheFull, FreeList
from .budget import CacheDoesNotFit
from .sequence_cache import PAGE_TOKENS, KVLayerView, SequenceCache, StateLayerView, pages_for
