"""What a mixer may ask of the cache manager for one cache slot."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values per token, in pages.  ``window`` W: only the last W keys
    of a sequence are ever read, so pages that a window has passed are given
    back.  None: all keys are kept while the request lives.  ``block_size``:
    tokens per page if the mixer wants a page size of its own (None: the
    engine's).  Slots with equal specs share a group: one pool, one table per
    request."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    block_size: Optional[int] = None


@dataclass(frozen=True)
class StateSpec:
    """State of fixed size per request (e.g. a recurrent mixer's), kept in a slot
    that the request holds from admission to its end.  A fresh request's slot is
    zeroed."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32
