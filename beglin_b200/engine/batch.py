"""One step's batch: for each request its next tokens, laid out as token rows in request order.

The reference's ragged step takes columns (token id, slot, position), consecutive columns of one
slot being a prompt portion (qwen_infer.c:2064-2068, :20626-20630).  A `StepBatch` holds the same
as device arrays, plus the block tables of the live requests and the rows whose logits are wanted.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch


@dataclass
class Entry:
    """A request's part of a step: its next tokens and the places among them whose logits are
    wanted."""
    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


class StepBatch:
    def __init__(self, entries: Sequence[Entry], starts: Sequence[int], device, cache=None):
        """`starts[i]` is the position of the first token of entry i (the request's length so far)."""
        self.entries = list(entries)
        self.device = torch.device(device)
        self.n_req = len(self.entries)
        ids: List[int] = []
        pos: List[int] = []
        req: List[int] = []
        rows: List[int] = []
        self.row_start: List[int] = []
        for i, (e, s) in enumerate(zip(self.entries, starts)):
            self.row_start.append(len(ids))
            n = len(e.tokens)
            ids.extend(int(t) for t in e.tokens)
            pos.extend(range(s, s + n))
            req.extend([i] * n)
            rows.extend(self.row_start[-1] + int(w) for w in e.want)
        self.n_rows = len(ids)
        self.starts = list(starts)
        self.lens = [len(e.tokens) for e in self.entries]
        self.max_position = max(pos) if pos else 0
        self.decode_only = all(n == 1 for n in self.lens)      # every request brings a single token
        self.n_logit_rows = len(rows)
        self.token_ids = self._to_device(np.asarray(ids, dtype=np.int32))
        self.positions = self._to_device(np.asarray(pos, dtype=np.int32))
        self.row_req = self._to_device(np.asarray(req, dtype=np.int32))
        self.logit_rows = self._to_device(np.asarray(rows, dtype=np.int32)) if rows else None
        self.block_tables: Dict[int, torch.Tensor] = {}
        self.slots: Optional[torch.Tensor] = None
        if cache is not None:
            rids = [e.rid for e in self.entries]
            for gi in range(len(cache.kv_groups)):
                self.block_tables[gi] = self._to_device(cache.block_table(gi, rids))
            self.slots = self._to_device(cache.slot_ids(rids))
        self.scratch: Dict[object, object] = {}       # per-step tables made by parts (rotary tables)
        self._qblk: Dict[int, Tuple[torch.Tensor, int]] = {}

    def _to_device(self, a: np.ndarray) -> torch.Tensor:
        t = torch.from_numpy(np.ascontiguousarray(a))
        if self.device.type == "cuda":
            return t.pin_memory().to(self.device, non_blocking=True)
        return t

    def query_blocks(self, bq: int) -> Tuple[torch.Tensor, int]:
        """Rows cut into blocks of at most `bq` consecutive rows of one request: int32 [n, 3] of
        (request, first row, number of rows)."""
        hit = self._qblk.get(bq)
        if hit is None:
            blocks = []
            for i, (r0, n) in enumerate(zip(self.row_start, self.lens)):
                for b in range(0, n, bq):
                    blocks.append((i, r0 + b, min(bq, n - b)))
            arr = np.asarray(blocks, dtype=np.int32).reshape(-1, 3)
            hit = (self._to_device(arr), len(blocks))
            self._qblk[bq] = hit
        return hit
