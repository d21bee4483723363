"""What a mixer asks of the cache for one execution of its layer."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class KVNeed:
    """Keys and values of every position (``window`` None) or of the last ``window`` positions."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class CacheNeeds:
    """``kv``: paged keys and values, or None.  ``state_elems``: float32 numbers of fixed-size
    state per sequence (0 for none); the state is zero when a sequence starts."""
    kv: Optional[KVNeed] = None
    state_elems: int = 0
