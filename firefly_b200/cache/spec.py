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
    engine's).  ``planes``: 2 = a plane of keys and a plane of values per page; 1 = one
    vector per token that serves as key and as value (a mixer that caches a latent
    vector).  Slots with equal specs share a group: one pool, one table per request."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    block_size: Optional[int] = None
    planes: int = 2


@dataclass(frozen=True)
class StateSpec:
    """State of fixed size per request (e.g. a recurrent mixer's), kept in a slot
    that the request holds from admission to its end.  A fresh request's slot is
    zeroed."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


SUB_SLOT_STRIDE = 1 << 20


def sub_slot(slot: int, k: int) -> int:
    """The id of the k-th cache of a mixer that keeps several (a mixer made of mixers: its ``cache_spec()`` is a
    tuple, one spec per inner mixer).  A run's own slot ids stay below ``SUB_SLOT_STRIDE``."""
    if not (0 <= slot < SUB_SLOT_STRIDE):
        raise ValueError(f"cache slot {slot} out of range")
    return slot + (k + 1) * SUB_SLOT_STRIDE


FILTER_SUB_SLOT = 63


def filter_slot(slot: int) -> int:
    """The id of the state that a block's input filter keeps beside its mixer's cache (a mixer made of mixers uses
    the sub-slots from 0 up)."""
    return sub_slot(slot, FILTER_SUB_SLOT)
