"""Decoding steps as a CUDA graph.

A step in which every request brings exactly one token has fixed shapes, so the whole step (embedding,
every layer's kernels, the head and the sampling kernel) is captured once per batch size and
replayed.  What changes from step to step is data in fixed device buffers: token ids, positions, block
tables, state slots, temperatures and uniform numbers.  The sampled tokens are also written back
into the token buffer on the device, so a caller that does not need them on the host can decode
without a round trip.

A graph stands for a batch of up to `n` requests, n one of `BUCKETS`: a step of fewer requests pads
the batch with rows that belong to nobody (token 0 at position 0, keys, values and state written to
the cache manager's spare page and spare slot, results dropped), so that requests which end one by
one go through at most a handful of graphs.

The attention kernels are launched for the context limit, not for the longest live request: the
float32 kernel cuts the keys at fixed positions, so a replayed float32 step computes every row
bitwise as the uncaptured step function does; the bfloat16 decoding kernel spreads a request's keys
over a number of CTAs that depends on the batch's size and the context limit, so there a replayed
step agrees with the uncaptured one up to rounding only.
"""
from __future__ import annotations

from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheError, OutOfPages
from ..csrc import ops
from .capture import no_collection


BUCKETS = (1, 2, 4, 8, 16, 32, 64)


def bucket(n: int) -> int:
    """The batch size of the graph that serves a step of n requests: the next of BUCKETS, and beyond
    the largest the next multiple of it."""
    for b in BUCKETS:
        if n <= b:
            return b
    top = BUCKETS[-1]
    return -(-n // top) * top


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
        self.meta = torch.zeros((3, n), dtype=torch.int32).pin_memory()          # positions, slots, live rows
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
        self.advance = torch.ones(n, dtype=torch.int32, device=dev)      # 1 for a live row, 0 for a row that pads
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
        # the sampled tokens become the next step's input and the positions move on inside the sampling kernel, so
        # the next step of the same requests needs no upload and the graph holds no kernel but the package's own
        ops.sample(logits, self.temperature, self.uniform, self.out_tokens, feed_tokens=b.token_ids,
                   feed_positions=b.positions, advance=self.advance)
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
            # Warm-up outside the capture (library handles, allocations).  The replay that follows runs the
            # same step again: keys and values are written twice with the same contents, and state of fixed
            # size, which a mixer reads, changes and writes, is put back as it was.
            saved_state = self.engine.cache.snapshot_state()
            self._body()
            self.engine.cache.restore_state(saved_state)
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
        """Upload the block tables that differ from what the device holds; returns the bytes sent.  The
        rows beyond the live requests hold the spare page at position 0 and nothing else."""
        cache, sent, m = self.engine.cache, 0, len(rids)
        for gi, h in st.tables.items():
            table = np.full((self.n, cache.max_pages), -1, dtype=np.int32)
            table[:m] = cache.block_table(gi, rids)
            table[m:, 0] = cache.dump_page
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
        cache = self.engine.cache
        if self._ahead is None or not all(cache.has(r) for r in rids) or self._ahead[0] != cache.identity(rids):
            return False
        return all(cache.length(r) == p for r, p in zip(rids, self._ahead[1]))

    def step(self, rids: Sequence[Hashable], tokens: Optional[Sequence[int]], temperatures: Optional[Sequence[float]] = None,
             uniforms: Optional[Sequence[float]] = None, read_back: bool = True):
        """One decoding step for `rids` (all live, pages reserved by the caller for one more position
        each).  `tokens` None means: feed what the previous replay sampled (kept on the device).
        Returns the sampled tokens as a list (read_back) or the device tensor.  Only what changed since
        the last step is uploaded: positions advance on the device, block tables change when a request
        gets a new page."""
        cache, n, b = self.engine.cache, self.n, self.batch
        m = len(rids)
        assert 1 <= m <= n
        st = self.ring[self.turn]
        self.turn = (self.turn + 1) % self.RING
        if st.event is not None:
            st.event.synchronize()             # the device has read this set's last contents
        sent = 0
        positions = [cache.length(r) for r in rids]
        key = cache.identity(rids)             # a request that ended and one that began under its name differ
        if key != self._rids or positions != self._positions:
            meta = st.meta.numpy()
            meta[0, :m], meta[0, m:] = positions, 0
            meta[1, :m], meta[1, m:] = cache.slot_ids(rids), cache.dump_slot
            meta[2, :m], meta[2, m:] = 1, 0
            b.positions.copy_(st.meta[0], non_blocking=True)
            b.slots.copy_(st.meta[1], non_blocking=True)
            self.advance.copy_(st.meta[2], non_blocking=True)
            sent += 12 * n
            self._rids = key
        fed = tokens is not None and read_back     # the copies in and out are part of the replayed graph
        if fed:
            self.h_in_np[:m] = tokens              # safe: the last fed step was waited for before it returned
            self.h_in_np[m:] = 0
            sent += 4 * n
        elif tokens is not None:
            h = st.tokens.numpy()
            h[:m], h[m:] = list(tokens), 0
            b.token_ids.copy_(st.tokens, non_blocking=True)
            sent += 4 * n
        if temperatures is not None and any(t > 0.0 for t in temperatures):
            f = st.floats.numpy()
            f[0, :m], f[0, m:] = list(temperatures), 0.0
            f[1, :m], f[1, m:] = list(uniforms), 0.0
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
            return self.h_out[:m].tolist()
        return self.out_tokens[:m]
