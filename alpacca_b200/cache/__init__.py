from .pool import CacheFull, IdPool
from .store import PAGE_SIZE, KVGroup, KVLayerView, SequenceCache, StateGroup, StateLayerView

__all__ = ["CacheFull", "IdPool", "PAGE_SIZE", "KVGroup", "KVLayerView", "SequenceCache", "StateGroup",
           "StateLayerView"]
