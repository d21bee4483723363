"""What a mixer asks of the cache for one execution of its layer."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class KVNeed:
    """Keys and values of every position (``window`` None) or of the last ``window`` positions.
    ``v_head_dim``: the size of a value head where it is not the keys' (None: the same); ``v_heads``: the
    number of value heads where it is not the keys' (a cache that keeps one compressed row per position
    asks for one key head and no value head: ``v_heads=0``)."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    v_head_dim: Optional[int] = None
    v_heads: Optional[int] = None

    @property
    def value_shape(self):
        """(heads, head size) of what a position keeps as values."""
        return (self.n_kv_heads if self.v_heads is None else self.v_heads,
                self.head_dim if self.v_head_dim is None else self.v_head_dim)


@dataclass(frozen=True)
class CacheNeeds:
    """``kv``: paged keys and values, or None.  ``state_elems``: numbers of fixed-size state per sequence
    (0 for none), kept as ``state_dtype`` ("float32", "bfloat16", or "engine" for the engine's own dtype);
    the state is zero when a sequence starts."""
    kv: Optional[KVNeed] = None
    state_elems: int = 0
    state_dtype: str = "float32"
