"""What a mixer asks of the cache manager, and what it is handed back each step.

A mixer's class method `cache_need(spec)` returns one of the needs below (or None).  Stages whose
needs are equal share a group of the cache manager: one page pool and one block table per request
for paged keys and values, one slab of slots for per-request state of fixed size.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values of every position (window None) or of the last `window` positions."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class FixedStateNeed:
    """A tensor of this shape per request, zero when the request starts, kept between steps."""
    shape: Tuple[int, ...]
    dtype: str = "float32"


@dataclass
class PagedKVView:
    """One stage's pages, [num_pages, 2, n_kv_heads, page_size, head_dim] (2 = keys, values), and
    the step's block table [requests, max_pages] (int32, -1 where no page is held)."""
    pool: torch.Tensor
    block_table: torch.Tensor
    page_size: int
    window: Optional[int]


@dataclass
class FixedStateView:
    """One stage's state slab [slots, *shape] and the step's slot of each request [requests]."""
    state: torch.Tensor
    slots: torch.Tensor
