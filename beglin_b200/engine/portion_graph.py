"""Prompt portions of one request as a CUDA graph.

A step that brings `rows` tokens of ONE request and wants the logits of `wanted` places has fixed shapes
whatever the request and wherever in its context the portion lies: a long prompt that the scheduler cuts
into portions of the token budget, or prompts run whole at a length that comes again, repeat one such
shape.  The step (embedding, every layer's kernels and library products, the final norm and the head) is
captured once per shape and replayed.  What changes from step to step is data in ONE fixed device buffer
(token ids, positions, the wanted rows, the state slot and the block tables), brought up to date with one
copy from pinned host memory.  The host then launches one graph instead of some three hundred kernels, so
the device never waits for it: at the layer sizes of Qwen2.5-1.5B launching a portion kernel by kernel
keeps the host busy for 4 ms, and the first kernels of a step are shorter than their launches.

The kernels and their arguments are those of the uncaptured step, so a replayed portion computes every
row as `Engine.step` does without a graph; `bound` (the largest position the shape may reach) only sizes
the scratch of the attention kernels that cut the keys into ranges at fixed positions.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from ..csrc import ops
from .batch import ALIGN
from .capture import no_collection


class _StaticPortion:
    """What the model's parts read from a step batch, for `rows` consecutive tokens of one request, with
    fixed device buffers behind it."""

    def __init__(self, rows: int, wanted: int, bound: int, cache, device):
        self.n_rows, self.n_req = rows, 1
        self.device = device
        self.entries: list = []
        self.row_start, self.lens = [0], [rows]
        self.starts = None                     # differs between replays: nothing on the host may depend on it
        self.decode_only = False
        self.implicit_blocks = False
        self.n_logit_rows = wanted
        self.max_position = bound
        self.scratch: Dict[object, object] = {}
        groups = len(cache.kv_groups)
        sizes = [("token_ids", rows), ("positions", rows), ("logit_rows", wanted), ("slots", 1)] + \
                [(("block_table", gi), cache.max_pages) for gi in range(groups)]
        self.offsets, total = {}, 0
        for name, n in sizes:
            self.offsets[name] = (total, n)
            total += -(-max(n, 1) // ALIGN) * ALIGN
        self.host = torch.zeros(total, dtype=torch.int32).pin_memory()
        self.host_np = self.host.numpy()
        self.buf = torch.zeros(total, dtype=torch.int32, device=device)
        view = lambda name: self.buf[self.offsets[name][0]:self.offsets[name][0] + self.offsets[name][1]]
        self.token_ids, self.positions, self.slots = view("token_ids"), view("positions"), view("slots")
        self.logit_rows = view("logit_rows") if wanted else None
        self.row_req = torch.zeros(rows, dtype=torch.int32, device=device)
        self.block_tables = {gi: view(("block_table", gi)).view(1, cache.max_pages) for gi in range(groups)}
        self._qblk: Dict[int, Tuple[torch.Tensor, int]] = {}

    def fill(self, name, values: np.ndarray) -> None:
        lo, n = self.offsets[name]
        self.host_np[lo:lo + n] = values

    def query_blocks(self, bq: int) -> Tuple[torch.Tensor, int]:
        hit = self._qblk.get(bq)
        if hit is None:
            first = np.arange(0, self.n_rows, bq, dtype=np.int32)
            arr = np.stack([np.zeros(first.size, dtype=np.int32), first,
                            np.minimum(bq, self.n_rows - first).astype(np.int32)], axis=1)
            hit = self._qblk[bq] = (torch.from_numpy(arr).to(self.device), int(arr.shape[0]))
        return hit


class PortionGraph:
    def __init__(self, engine, rows: int, wanted: int, bound: int):
        self.engine, self.rows, self.wanted, self.bound = engine, rows, wanted, bound
        self.batch = _StaticPortion(rows, wanted, bound, engine.cache, engine.device)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.launches = 0
        self.taken: Optional[torch.cuda.Event] = None      # the device has read the pinned buffer's last contents

    def _body(self) -> None:
        self.batch.scratch.clear()
        self.logits = self.engine.model.forward(self.batch, self.engine.cache)

    def _capture(self) -> None:
        side = torch.cuda.Stream(device=self.engine.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            # warm-up outside the capture (library handles, allocations); it writes the same keys and values
            # the replay will, and state of fixed size is put back as it was
            saved_state = self.engine.cache.snapshot_state()
            self._body()
            self.engine.cache.restore_state(saved_state)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        before = ops.launch_count()
        g = torch.cuda.CUDAGraph()
        with no_collection(), torch.cuda.graph(g):
            self._body()
        self.launches = ops.launch_count() - before
        self.graph = g

    def step(self, entry, start: int) -> Optional[torch.Tensor]:
        """Run the portion `entry` (its request's pages reserved by the caller) whose first token stands at
        position `start`.  Returns the logits of the wanted places, in a tensor of the caller's own."""
        b, cache = self.batch, self.engine.cache
        assert len(entry.tokens) == self.rows and len(entry.want) == self.wanted
        assert start + self.rows - 1 <= self.bound
        if self.taken is not None:
            self.taken.synchronize()
        ids = entry.ids()
        if ids.size and (ids.min() < 0 or ids.max() > 0x7fffffff):
            ids = np.where((ids < 0) | (ids > 0x7fffffff), -1, ids)          # the embedding kernel reports these
        b.fill("token_ids", ids.astype(np.int32))
        b.fill("positions", np.arange(start, start + self.rows, dtype=np.int32))
        if self.wanted:
            b.fill("logit_rows", np.asarray([int(w) for w in entry.want], dtype=np.int32))
        b.fill("slots", cache.slot_ids([entry.rid]))
        for gi in range(len(cache.kv_groups)):
            b.fill(("block_table", gi), cache.block_table(gi, [entry.rid]).reshape(-1))
        b.buf.copy_(b.host, non_blocking=True)
        self.taken = torch.cuda.Event()
        self.taken.record()
        if self.graph is None:
            self._capture()
        self.graph.replay()
        ops.count_launches(self.launches)
        return self.logits.clone() if self.logits is not None else None


class PortionGraphs:
    """The portion graphs of an engine: a shape is captured when it comes for the second time, and the
    shapes used least recently are dropped beyond `keep` graphs (each holds its step's activations)."""

    BOUND_STEP = 4096          # `bound` grows in steps of this many positions

    def __init__(self, engine, min_rows: int = 256, max_wanted: int = 8, keep: int = 4):
        self.engine, self.min_rows, self.max_wanted, self.keep = engine, min_rows, max_wanted, keep
        self.graphs: Dict[tuple, PortionGraph] = {}
        self.seen: List[tuple] = []
        self.replays = 0

    def key_of(self, ents, starts) -> Optional[tuple]:
        """The shape of a step that a graph can stand for, or None."""
        if len(ents) != 1:
            return None
        rows, wanted = len(ents[0].tokens), len(ents[0].want)
        if rows < self.min_rows or wanted > self.max_wanted:
            return None
        limit = self.engine.cache.max_context - 1
        bound = min(limit, -(-(starts[0] + rows) // self.BOUND_STEP) * self.BOUND_STEP - 1)
        return rows, wanted, bound

    def get(self, key) -> Optional[PortionGraph]:
        g = self.graphs.get(key)
        if g is None:
            if key not in self.seen:           # first sighting: remember it, run the step kernel by kernel
                self.seen.append(key)
                del self.seen[:-16]
                return None
            while len(self.graphs) >= self.keep:
                del self.graphs[next(iter(self.graphs))]
            g = PortionGraph(self.engine, *key)
        else:
            del self.graphs[key]               # moved to the end: used most recently
        self.graphs[key] = g
        return g

    def step(self, g: PortionGraph, entry, start: int) -> Optional[torch.Tensor]:
        self.replays += 1
        return g.step(entry, start)
