"""What a mixer asks of the cache manager for one cache entry."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values of every position (window None) or of the last `window`
    positions, in pages [num_pages, num_kv_heads, page_size, head_dim]."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """A state of fixed size per request, in a slot: [num_slots, *shape].
    `dtype` None means the activation type. A slot is zeroed when a request opens."""

    shape: tuple
    dtype: object = None
