"""The cache manager: pages of keys and values with a block table per request, and slots for
per-request state of fixed size.

The reference keeps a contiguous cache per request slot, statically sized, gives a slot back the
moment its request ends and never clears it between users (qwen_infer.c:1775-1807, :2032-2037,
:2176-2179).  Pages replace the static slots here; the rest is kept: what a finished request held
is free at once for the next one, and nothing is cleared, since every position is written before it
is read.

Stages of the model whose mixers have equal needs form a group.  A group of paged keys and values
has one pool of pages (shared by its stages: page p of every stage of the group belongs to the same
request and the same positions) and one block table per request.  A group with a window gives back
the pages that lie wholly behind the window as a request advances.  A group of fixed state has one
slab [stages, slots, ...]; a request's slot is zeroed when the request starts.

All accounting is host code on plain Python and numpy and is tested without a GPU; only `allocate`
makes device tensors.
"""
from __future__ import annotations

from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..parts.cache_need import FixedStateNeed, FixedStateView, PagedKVNeed, PagedKVView


class OutOfPages(RuntimeError):
    """A reservation needs more free pages than a pool has.  Nothing was changed."""


class CacheError(RuntimeError):
    pass


class PagePool:
    """Free list of page numbers.  Last freed, first reused, so reuse shows up early."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._held = bytearray(num_pages)

    @property
    def num_free(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> List[int]:
        if n > len(self._free):
            raise OutOfPages(f"{n} pages wanted, {len(self._free)} of {self.num_pages} free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = 1
        return out

    def free(self, pages: Sequence[int]) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages or not self._held[p]:
                raise CacheError(f"page {p} freed but not held")
            self._held[p] = 0
            self._free.append(p)

    def check(self) -> None:
        """No page lost or listed twice."""
        if len(set(self._free)) != len(self._free):
            raise CacheError("a page is on the free list twice")
        if len(self._free) + sum(self._held) != self.num_pages:
            raise CacheError("pages lost: free + held != total")
        for p in self._free:
            if self._held[p]:
                raise CacheError(f"page {p} is both free and held")


class _KVGroup:
    def __init__(self, need: PagedKVNeed, stages: List[int], num_pages: int):
        self.need, self.stages = need, stages
        self.pool = PagePool(num_pages)
        self.tables: Dict[Hashable, List[int]] = {}     # request -> page of each page index, -1 if none
        self.device_pool: Optional[torch.Tensor] = None  # [stages, pages, 2, nkv, page, hd]

    def first_needed_page(self, first_query_pos: int, page_size: int) -> int:
        if self.need.window is None:
            return 0
        lo = max(0, first_query_pos - self.need.window + 1)
        return lo // page_size


class _StateGroup:
    def __init__(self, need: FixedStateNeed, stages: List[int]):
        self.need, self.stages = need, stages
        self.slab: Optional[torch.Tensor] = None         # [stages, slots, *shape]


class CacheManager:
    def __init__(self, needs: Sequence[Optional[object]], page_size: int, num_pages: int, max_requests: int,
                 max_context: Optional[int] = None):
        """`needs[i]` is the need of stage i of the model's run order (None: no cache of its own).
        Every paged group gets `num_pages` pages of `page_size` positions."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size, self.num_pages, self.max_requests = page_size, num_pages, max_requests
        self.max_context = max_context if max_context is not None else num_pages * page_size
        self.max_pages = -(-self.max_context // page_size)
        self.kv_groups: List[_KVGroup] = []
        self.state_groups: List[_StateGroup] = []
        self.stage_group: Dict[int, tuple] = {}          # stage -> ("kv" | "state", group index, index in group)
        for stage, need in enumerate(needs):
            if need is None:
                continue
            if isinstance(need, PagedKVNeed):
                groups, kind, make = self.kv_groups, "kv", lambda n: _KVGroup(n, [], num_pages)
            elif isinstance(need, FixedStateNeed):
                groups, kind, make = self.state_groups, "state", lambda n: _StateGroup(n, [])
            else:
                raise TypeError(f"stage {stage}: unknown cache need {need!r}")
            for gi, g in enumerate(groups):
                if g.need == need:
                    break
            else:
                groups.append(make(need))
                gi = len(groups) - 1
            self.stage_group[stage] = (kind, gi, len(groups[gi].stages))
            groups[gi].stages.append(stage)
        self.lengths: Dict[Hashable, int] = {}
        self.slots: Dict[Hashable, int] = {}
        self._free_slots: List[int] = list(range(max_requests - 1, -1, -1))
        # Every start of a request gets a number of its own, so that whoever remembers what the device holds
        # for a request (a replayed graph's block tables and positions) can tell a request from a later one
        # of the same name.
        self.births: Dict[Hashable, int] = {}
        self._born = 0
        # One page and one state slot more than are ever handed out: rows that pad a batch of fixed shape
        # write their keys, values and state there, where no request reads.
        self.dump_page = num_pages
        self.dump_slot = max_requests

    # ---------------------------------------------------------------- device side
    def allocate(self, device, dtype: torch.dtype) -> None:
        for g in self.kv_groups:
            g.device_pool = torch.empty((len(g.stages), self.num_pages + 1, 2, g.need.n_kv_heads, self.page_size,
                                         g.need.head_dim), dtype=dtype, device=device)
            g.device_pool[:, self.dump_page].zero_()
        for g in self.state_groups:
            g.slab = torch.zeros((len(g.stages), self.max_requests + 1) + tuple(g.need.shape),
                                 dtype=getattr(torch, g.need.dtype), device=device)

    def snapshot_state(self) -> list:
        """Copies of the fixed-state slabs, for a caller that has to run a step twice (a warm-up before a
        stream capture) and must not advance the state twice."""
        return [g.slab.clone() if g.slab is not None else None for g in self.state_groups]

    def restore_state(self, saved: list) -> None:
        for g, s in zip(self.state_groups, saved):
            if s is not None:
                g.slab.copy_(s)

    def device_bytes(self) -> int:
        total = 0
        for g in self.kv_groups:
            if g.device_pool is not None:
                total += g.device_pool.numel() * g.device_pool.element_size()
        for g in self.state_groups:
            if g.slab is not None:
                total += g.slab.numel() * g.slab.element_size()
        return total

    # ---------------------------------------------------------------- requests
    def has(self, rid: Hashable) -> bool:
        return rid in self.lengths

    def length(self, rid: Hashable) -> int:
        return self.lengths[rid]

    def live(self) -> List[Hashable]:
        return list(self.lengths)

    def can_add(self) -> bool:
        return bool(self._free_slots)

    def add_request(self, rid: Hashable) -> int:
        if rid in self.lengths:
            raise CacheError(f"request {rid!r} is already live")
        if not self._free_slots:
            raise CacheError(f"all {self.max_requests} request slots are taken")
        slot = self._free_slots.pop()
        self.lengths[rid] = 0
        self.slots[rid] = slot
        self._born += 1
        self.births[rid] = self._born
        for g in self.kv_groups:
            g.tables[rid] = []
        for g in self.state_groups:
            if g.slab is not None:
                g.slab[:, slot].zero_()
        return slot

    def release(self, rid: Hashable) -> None:
        """Give back everything the request holds."""
        if rid not in self.lengths:
            raise CacheError(f"request {rid!r} is not live")
        for g in self.kv_groups:
            g.pool.free([p for p in g.tables.pop(rid) if p >= 0])
        self._free_slots.append(self.slots.pop(rid))
        del self.lengths[rid]
        del self.births[rid]

    def identity(self, rids: Sequence[Hashable]) -> tuple:
        """(request, number of its start) for each: equal only for the same live requests."""
        return tuple((r, self.births[r]) for r in rids)

    def trim(self, rids: Sequence[Hashable]) -> None:
        """Give back the pages that lie beyond each request's recorded length: what a reservation took for
        a step that did not happen."""
        for rid in rids:
            if rid not in self.lengths:
                continue
            keep = -(-self.lengths[rid] // self.page_size)
            for g in self.kv_groups:
                table = g.tables[rid]
                if len(table) > keep:
                    g.pool.free([p for p in table[keep:] if p >= 0])
                    del table[keep:]

    # ---------------------------------------------------------------- pages
    def _plan(self, g: _KVGroup, rid: Hashable, new_len: int, first_query_pos: int):
        """(page indexes to give back, number of page indexes to add) for one group."""
        table = g.tables[rid]
        first = g.first_needed_page(first_query_pos, self.page_size)
        drop = [i for i in range(min(first, len(table))) if table[i] >= 0] if first > 0 else ()
        want_pages = -(-new_len // self.page_size)
        add = max(0, want_pages - len(table))
        return drop, add

    def _plans(self, plan: Sequence[tuple]):
        """For every group, the (give back, add) of every entry of the plan."""
        out, ps = [], self.page_size
        for g in self.kv_groups:
            if g.need.window is None:          # nothing is ever given back before the request ends
                tables = g.tables
                out.append([((), max(0, -(-new_len // ps) - len(tables[rid]))) for rid, new_len in plan])
            else:
                out.append([self._plan(g, rid, new_len, self.lengths[rid]) for rid, new_len in plan])
        return out

    @staticmethod
    def _short(groups, plans) -> int:
        short = 0
        for g, per_request in zip(groups, plans):
            need = sum(add - len(drop) for drop, add in per_request)
            short = max(short, need - g.pool.num_free)
        return max(0, short)

    def pages_short(self, plan: Sequence[tuple]) -> int:
        """How many pages the fullest pool lacks for `plan` = [(request, new length), ...], counting
        what the plan itself gives back.  0 means the plan fits."""
        return self._short(self.kv_groups, self._plans(plan))

    def reserve(self, plan: Sequence[tuple]) -> None:
        """Make room for every (request, new length) of a step, or raise OutOfPages and change
        nothing.  The first new position of a request is its current length; a windowed group first
        gives back the pages wholly behind that position's window."""
        for rid, new_len in plan:
            if rid not in self.lengths:
                raise CacheError(f"request {rid!r} is not live")
            if new_len > self.max_context:
                raise CacheError(f"request {rid!r} would hold {new_len} positions, more than the context "
                                 f"limit {self.max_context}")
            if new_len < self.lengths[rid]:
                raise CacheError(f"request {rid!r} cannot shrink from {self.lengths[rid]} to {new_len}")
        plans = self._plans(plan)
        short = self._short(self.kv_groups, plans)
        if short:
            raise OutOfPages(f"the step needs {short} more pages than are free")
        for g, per_request in zip(self.kv_groups, plans):
            for (rid, _), (drop, _) in zip(plan, per_request):      # first everything that is given back,
                if drop:
                    table = g.tables[rid]
                    g.pool.free([table[i] for i in drop])
                    for i in drop:
                        table[i] = -1
            for (rid, _), (_, add) in zip(plan, per_request):       # then what is added (a table's length does not change above)
                if add:
                    g.tables[rid].extend(g.pool.alloc(add))

    def commit(self, plan: Sequence[tuple]) -> None:
        """Record the new lengths after the step has run."""
        for rid, new_len in plan:
            self.lengths[rid] = new_len

    def pages_held(self, rid: Hashable) -> int:
        return max((sum(1 for p in g.tables[rid] if p >= 0) for g in self.kv_groups), default=0)

    def free_pages(self) -> int:
        return min((g.pool.num_free for g in self.kv_groups), default=self.num_pages)

    def check(self) -> None:
        """Invariants: no page lost, held by two requests, or free while held."""
        for g in self.kv_groups:
            g.pool.check()
            seen = set()
            for rid, table in g.tables.items():
                for p in table:
                    if p < 0:
                        continue
                    if p in seen:
                        raise CacheError(f"page {p} is held twice")
                    seen.add(p)
            if len(seen) + g.pool.num_free != g.pool.num_pages:
                raise CacheError("pages held by requests + free != total")
        if len(set(self.slots.values())) != len(self.slots):
            raise CacheError("a state slot is held twice")
        if len(self.slots) + len(self._free_slots) != self.max_requests:
            raise CacheError("state slots lost")

    # ---------------------------------------------------------------- what a step reads
    def block_table(self, group: int, rids: Sequence[Hashable]) -> np.ndarray:
        out = np.full((len(rids), self.max_pages), -1, dtype=np.int32)
        g = self.kv_groups[group]
        for i, rid in enumerate(rids):
            t = g.tables[rid]
            out[i, :len(t)] = t
        return out

    def slot_ids(self, rids: Sequence[Hashable]) -> np.ndarray:
        return np.asarray([self.slots[r] for r in rids], dtype=np.int32)

    def view(self, stage: int, batch):
        """The cache view of one stage for a step: its pages and the step's block table, or its state
        slab and the step's slots."""
        kind, gi, idx = self.stage_group[stage]
        if kind == "kv":
            g = self.kv_groups[gi]
            return PagedKVView(g.device_pool[idx], batch.block_tables[gi], self.page_size, g.need.window)
        g = self.state_groups[gi]
        return FixedStateView(g.slab[idx], batch.slots)
