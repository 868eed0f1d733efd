"""Decoding steps as a CUDA graph.

A step in which every request brings exactly one token has fixed shapes, so the whole step (embedding,
every layer's kernels, the head and the sampling kernel) is captured once per batch size and
replayed.  What changes from step to step is data in fixed device buffers: token ids, positions, block
tables, state slots, temperatures and uniform numbers.  The sampled tokens are also written back
into the token buffer on the device, so a caller that does not need them on the host can decode
without a round trip.

The attention kernel is launched for as many key splits as the context limit has; splits beyond a
request's length return at once.  The split boundaries are fixed positions, so a replayed step
computes every row exactly as the uncaptured step function does.
"""
from __future__ import annotations

from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheError, OutOfPages
from ..csrc import ops
from .capture import no_collection


class _StaticBatch:
    """What the model's parts read from a step batch, with fixed device buffers behind it."""

    def __init__(self, n: int, cache, device):
        self.n_rows = self.n_req = n
        self.device = device
        self.row_start = list(range(n))
        self.lens = [1] * n
        self.starts = [0] * n
        self.entries = []
        self.n_logit_rows = n
        self.decode_only = True
        self.implicit_blocks = True
        self.max_position = cache.max_context - 1
        i32 = dict(dtype=torch.int32, device=device)
        self.token_ids = torch.zeros(n, **i32)
        self.positions = torch.zeros(n, **i32)
        self.row_req = torch.arange(n, **i32)
        self.logit_rows = torch.arange(n, **i32)
        self.slots = torch.zeros(n, **i32)
        self.block_tables = {gi: torch.full((n, cache.max_pages), -1, **i32) for gi in range(len(cache.kv_groups))}
        self.scratch: Dict[object, object] = {}
        self._qblk = torch.stack([torch.arange(n), torch.arange(n), torch.ones(n, dtype=torch.long)], dim=1) \
            .to(torch.int32).to(device).contiguous()

    def query_blocks(self, bq: int) -> Tuple[Optional[torch.Tensor], int]:
        """Block i is row i of request i.  The decoding kernel knows that without a list (bq == 1 and
        every request brings one row), which spares it a dependent load; other kernels get the list."""
        return (None if bq == 1 and self.implicit_blocks else self._qblk), self.n_rows


class _Staging:
    """One set of pinned host buffers for a step's uploads, with an event that says when the device
    has taken them."""

    def __init__(self, n: int, cache):
        self.meta = torch.zeros((2, n), dtype=torch.int32).pin_memory()          # positions, slots
        self.tokens = torch.zeros(n, dtype=torch.int32).pin_memory()
        self.floats = torch.zeros((2, n), dtype=torch.float32).pin_memory()      # temperatures, uniforms
        self.tables = {gi: torch.zeros((n, cache.max_pages), dtype=torch.int32).pin_memory()
                       for gi in range(len(cache.kv_groups))}
        self.event: Optional[torch.cuda.Event] = None


class DecodeGraph:
    RING = 4          # the host may prepare this many steps ahead of the device

    def __init__(self, engine, n: int):
        self.engine, self.n = engine, n
        dev = engine.device
        cache = engine.cache
        self.batch = _StaticBatch(n, cache, dev)
        self.temperature = torch.zeros(n, dtype=torch.float32, device=dev)
        self.uniform = torch.zeros(n, dtype=torch.float32, device=dev)
        self.out_tokens = torch.zeros(n, dtype=torch.int32, device=dev)
        self.logits: Optional[torch.Tensor] = None
        self.ring = [_Staging(n, cache) for _ in range(self.RING)]
        self.turn = 0
        self.h_out = torch.zeros(n, dtype=torch.int32).pin_memory()
        self.h_in = torch.zeros(n, dtype=torch.int32).pin_memory()
        self.h_in_np = self.h_in.numpy()
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        # the same step with the host's tokens copied in at its head and the sampled ones copied out at its
        # tail, for a caller that feeds every step from the host and reads every result: one launch per step
        self.graph_fed: Optional[torch.cuda.CUDAGraph] = None
        self.launches = 0
        self.h2d_bytes = 0                     # bytes uploaded by the last step
        self._rids: Optional[tuple] = None     # what the device buffers describe
        self._positions: Optional[List[int]] = None
        self._tables: Dict[int, np.ndarray] = {}
        self._sampling = False
        self._ahead = None                     # ((rids), positions) whose pages and tables are in place already
        self._ahead_bytes = 0

    def _body(self) -> None:
        b = self.batch
        b.scratch.clear()
        logits = self.engine.model.forward(b, self.engine.cache)
        ops.sample(logits, self.temperature, self.uniform, self.out_tokens)
        b.token_ids.copy_(self.out_tokens)
        b.positions.add_(1)                    # the next step of the same requests needs no upload
        self.logits = logits

    def _body_fed(self) -> None:
        self.batch.token_ids.copy_(self.h_in, non_blocking=True)
        self._body()
        self.h_out.copy_(self.out_tokens, non_blocking=True)

    def _capture(self, fed: bool = False) -> None:
        body = self._body_fed if fed else self._body
        side = torch.cuda.Stream(device=self.engine.device)
        side.wait_stream(torch.cuda.current_stream())
        saved_tokens, saved_pos = self.batch.token_ids.clone(), self.batch.positions.clone()
        with torch.cuda.stream(side):
            self._body()                       # warm-up outside the capture (library handles, allocations)
            self.batch.token_ids.copy_(saved_tokens)
            self.batch.positions.copy_(saved_pos)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        before = ops.launch_count()
        g = torch.cuda.CUDAGraph()
        with no_collection(), torch.cuda.graph(g):
            body()
        self.launches = ops.launch_count() - before
        if fed:
            self.graph_fed = g
        else:
            self.graph = g

    def _upload_tables(self, rids, st) -> int:
        """Upload the block tables that differ from what the device holds; returns the bytes sent."""
        cache, sent = self.engine.cache, 0
        for gi, h in st.tables.items():
            table = cache.block_table(gi, rids)
            last = self._tables.get(gi)
            if last is None or not np.array_equal(last, table):
                h.copy_(torch.from_numpy(table))
                self.batch.block_tables[gi].copy_(h, non_blocking=True)
                self._tables[gi] = table
                sent += table.size * 4
        return sent

    def _look_ahead(self, key, rids) -> None:
        """While the device runs this step, do the host's part of the next step of the same requests: make
        room for one more position each and, when a request got a new page, upload its block table (the
        copy is queued behind this step's graph).  If the next call is for other requests, or there is no
        room, nothing is lost: that call does its own bookkeeping."""
        cache = self.engine.cache
        self._ahead, self._ahead_bytes = None, 0
        nxt = [p + 1 for p in self._positions]
        if any(n > cache.max_context for n in nxt):
            return
        try:
            cache.reserve(list(zip(rids, nxt)))
        except (OutOfPages, CacheError):
            return
        st = self.ring[self.turn]              # the staging set of the next call
        if st.event is not None:
            st.event.synchronize()
        sent = self._upload_tables(rids, st)
        if sent:
            st.event = torch.cuda.Event()
            st.event.record()
        self._ahead, self._ahead_bytes = (key, list(self._positions)), sent

    def prepared(self, rids: Sequence[Hashable]) -> bool:
        """Whether the last step has already made room for the next step of exactly these requests."""
        if self._ahead is None or self._ahead[0] != tuple(rids):
            return False
        cache = self.engine.cache
        return all(cache.length(r) == p for r, p in zip(rids, self._ahead[1]))

    def step(self, rids: Sequence[Hashable], tokens: Optional[Sequence[int]], temperatures: Optional[Sequence[float]] = None,
             uniforms: Optional[Sequence[float]] = None, read_back: bool = True):
        """One decoding step for `rids` (all live, pages reserved by the caller for one more position
        each).  `tokens` None means: feed what the previous replay sampled (kept on the device).
        Returns the sampled tokens as a list (read_back) or the device tensor.  Only what changed since
        the last step is uploaded: positions advance on the device, block tables change when a request
        gets a new page."""
        cache, n, b = self.engine.cache, self.n, self.batch
        assert len(rids) == n
        st = self.ring[self.turn]
        self.turn = (self.turn + 1) % self.RING
        if st.event is not None:
            st.event.synchronize()             # the device has read this set's last contents
        sent = 0
        positions = [cache.length(r) for r in rids]
        key = tuple(rids)
        if key != self._rids or positions != self._positions:
            st.meta[0] = torch.as_tensor(positions, dtype=torch.int32)
            st.meta[1] = torch.from_numpy(cache.slot_ids(rids))
            b.positions.copy_(st.meta[0], non_blocking=True)
            b.slots.copy_(st.meta[1], non_blocking=True)
            sent += 8 * n
            self._rids = key
        fed = tokens is not None and read_back     # the copies in and out are part of the replayed graph
        if fed:
            self.h_in_np[:] = tokens               # safe: the last fed step was waited for before it returned
            sent += 4 * n
        elif tokens is not None:
            st.tokens.copy_(torch.as_tensor(list(tokens), dtype=torch.int32))
            b.token_ids.copy_(st.tokens, non_blocking=True)
            sent += 4 * n
        if temperatures is not None and any(t > 0.0 for t in temperatures):
            st.floats[0] = torch.as_tensor(list(temperatures), dtype=torch.float32)
            st.floats[1] = torch.as_tensor(list(uniforms), dtype=torch.float32)
            self.temperature.copy_(st.floats[0], non_blocking=True)
            self.uniform.copy_(st.floats[1], non_blocking=True)
            sent += 8 * n
            self._sampling = True
        elif self._sampling:
            self.temperature.zero_()
            self._sampling = False
        if self._ahead != (key, positions):    # else the last step has brought the tables up to date already
            sent += self._upload_tables(rids, st)
        if sent > (4 * n if fed else 0):
            st.event = torch.cuda.Event()
            st.event.record()
        self.h2d_bytes = sent + self._ahead_bytes
        if fed:
            if self.graph_fed is None:
                self._capture(fed=True)
            self.graph_fed.replay()
        else:
            if self.graph is None:
                self._capture()
            self.graph.replay()
        ops.count_launches(self.launches)
        cache.commit([(r, p + 1) for r, p in zip(rids, positions)])
        self._positions = [p + 1 for p in positions]
        self._look_ahead(key, rids)
        if read_back:
            if not fed:
                self.h_out.copy_(self.out_tokens, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            return self.h_out.tolist()
        return self.out_tokens
