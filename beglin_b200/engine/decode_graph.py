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

from ..csrc import ops


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

    def query_blocks(self, bq: int) -> Tuple[torch.Tensor, int]:
        return self._qblk, self.n_rows


class DecodeGraph:
    def __init__(self, engine, n: int):
        self.engine, self.n = engine, n
        dev = engine.device
        cache = engine.cache
        self.batch = _StaticBatch(n, cache, dev)
        self.temperature = torch.zeros(n, dtype=torch.float32, device=dev)
        self.uniform = torch.zeros(n, dtype=torch.float32, device=dev)
        self.out_tokens = torch.zeros(n, dtype=torch.int32, device=dev)
        self.logits: Optional[torch.Tensor] = None
        # pinned staging: [positions | slots | tokens] and one block table per group
        self.h_meta = torch.zeros((3, n), dtype=torch.int32).pin_memory()
        self.h_float = torch.zeros((2, n), dtype=torch.float32).pin_memory()
        self.h_tables = {gi: torch.zeros((n, cache.max_pages), dtype=torch.int32).pin_memory()
                         for gi in range(len(cache.kv_groups))}
        self.h_out = torch.zeros(n, dtype=torch.int32).pin_memory()
        self.d_meta = torch.zeros((3, n), dtype=torch.int32, device=dev)
        self.d_float = torch.zeros((2, n), dtype=torch.float32, device=dev)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.launches = 0
        self._table_version: Dict[int, object] = {}

    def _body(self) -> None:
        b = self.batch
        b.positions.copy_(self.d_meta[0])
        b.slots.copy_(self.d_meta[1])
        b.scratch.clear()
        self.temperature.copy_(self.d_float[0])
        self.uniform.copy_(self.d_float[1])
        logits = self.engine.model.forward(b, self.engine.cache)
        ops.sample(logits, self.temperature, self.uniform, self.out_tokens)
        b.token_ids.copy_(self.out_tokens)
        self.logits = logits

    def _capture(self) -> None:
        side = torch.cuda.Stream(device=self.engine.device)
        side.wait_stream(torch.cuda.current_stream())
        saved = self.batch.token_ids.clone()
        with torch.cuda.stream(side):
            self._body()                       # warm-up outside the capture (library handles, allocations)
            self.batch.token_ids.copy_(saved)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        before = ops.launch_count()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._body()
        self.launches = ops.launch_count() - before
        self.graph = g

    def step(self, rids: Sequence[Hashable], tokens: Optional[Sequence[int]], temperatures: Optional[Sequence[float]] = None,
             uniforms: Optional[Sequence[float]] = None, read_back: bool = True):
        """One decoding step for `rids` (all live, pages reserved by the caller for one more position
        each).  `tokens` None means: feed what the previous replay sampled (kept on the device).
        Returns the sampled tokens as a list (read_back) or the device tensor."""
        eng, cache, n = self.engine, self.engine.cache, self.n
        assert len(rids) == n
        self.h_meta[0] = torch.as_tensor([cache.length(r) for r in rids], dtype=torch.int32)
        self.h_meta[1] = torch.from_numpy(cache.slot_ids(rids))
        if tokens is not None:
            self.h_meta[2] = torch.as_tensor(list(tokens), dtype=torch.int32)
        self.d_meta.copy_(self.h_meta, non_blocking=True)
        if tokens is not None:
            self.batch.token_ids.copy_(self.d_meta[2])
        if temperatures is not None:
            self.h_float[0] = torch.as_tensor(list(temperatures), dtype=torch.float32)
            self.h_float[1] = torch.as_tensor(list(uniforms), dtype=torch.float32)
            self.d_float.copy_(self.h_float, non_blocking=True)
        for gi, h in self.h_tables.items():
            h.copy_(torch.from_numpy(cache.block_table(gi, rids)))
            self.batch.block_tables[gi].copy_(h, non_blocking=True)
        if self.graph is None:
            self._capture()
        self.graph.replay()
        ops.count_launches(self.launches)
        cache.commit([(r, cache.length(r) + 1) for r in rids])
        if read_back:
            self.h_out.copy_(self.out_tokens, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            return self.h_out.tolist()
        return self.out_tokens
