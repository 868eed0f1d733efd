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

    def ids(self) -> np.ndarray:
        """The tokens as an int64 array, converted once."""
        a = self.__dict__.get("_ids")
        if a is None:
            a = self.__dict__["_ids"] = np.asarray(self.tokens, dtype=np.int64).reshape(-1)
        return a


ALIGN = 32      # every array of a step starts on a multiple of this many int32 values (128 bytes) of the one buffer


class StepBatch:
    def __init__(self, entries: Sequence[Entry], starts: Sequence[int], device, cache=None):
        """`starts[i]` is the position of the first token of entry i (the request's length so far).
        All the step's integer arrays are laid out in ONE host buffer and go to the device in one copy;
        the device arrays are views of it."""
        self.entries = list(entries)
        self.device = torch.device(device)
        self.n_req = len(self.entries)
        self.row_start: List[int] = []
        self.lens = [len(e.tokens) for e in self.entries]
        self.starts = [int(s) for s in starts]
        ids_parts, pos_parts, req_parts, rows = [], [], [], []
        n_rows = 0
        for i, (e, s, n) in enumerate(zip(self.entries, self.starts, self.lens)):
            self.row_start.append(n_rows)
            t64 = e.ids()
            if t64.size and (t64.min() < 0 or t64.max() > 0x7fffffff):
                t64 = np.where((t64 < 0) | (t64 > 0x7fffffff), -1, t64)      # the embedding kernel reports these
            ids_parts.append(t64.astype(np.int32))
            pos_parts.append(np.arange(s, s + n, dtype=np.int32))
            req_parts.append(np.full(n, i, dtype=np.int32))
            rows.extend(n_rows + int(w) for w in e.want)
            n_rows += n
        cat = lambda parts: np.concatenate(parts) if parts else np.zeros(0, dtype=np.int32)
        self.n_rows = n_rows
        self.max_position = max((s + n - 1 for s, n in zip(self.starts, self.lens) if n > 0), default=0)
        self.decode_only = all(n == 1 for n in self.lens)      # every request brings a single token
        self.n_logit_rows = len(rows)
        arrays = {"token_ids": cat(ids_parts), "positions": cat(pos_parts), "row_req": cat(req_parts)}
        if rows:
            arrays["logit_rows"] = np.asarray(rows, dtype=np.int32)
        if cache is not None:
            rids = [e.rid for e in self.entries]
            for gi in range(len(cache.kv_groups)):
                arrays[("block_table", gi)] = cache.block_table(gi, rids)
            arrays["slots"] = cache.slot_ids(rids)
        dev = self._to_device_packed(arrays)
        self.token_ids, self.positions, self.row_req = dev["token_ids"], dev["positions"], dev["row_req"]
        self.logit_rows = dev.get("logit_rows")
        self.block_tables: Dict[int, torch.Tensor] = {k[1]: v for k, v in dev.items() if isinstance(k, tuple)}
        self.slots: Optional[torch.Tensor] = dev.get("slots")
        self.scratch: Dict[object, object] = {}       # per-step tables made by parts (rotary tables)
        self._qblk: Dict[int, Tuple[torch.Tensor, int]] = {}

    def _to_device_packed(self, arrays: Dict[object, np.ndarray]) -> Dict[object, torch.Tensor]:
        """int32 arrays -> device tensors of the same shapes, through one buffer and one copy."""
        offsets, total = {}, 0
        for k, a in arrays.items():
            offsets[k] = total
            total += -(-a.size // ALIGN) * ALIGN
        host = np.zeros(max(total, ALIGN), dtype=np.int32)
        for k, a in arrays.items():
            host[offsets[k]:offsets[k] + a.size] = np.asarray(a, dtype=np.int32).reshape(-1)
        buf = self._to_device(host)
        return {k: buf[offsets[k]:offsets[k] + a.size].view(a.shape) for k, a in arrays.items()}

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
            parts = []
            for i, (r0, n) in enumerate(zip(self.row_start, self.lens)):
                first = np.arange(0, n, bq, dtype=np.int32)
                parts.append(np.stack([np.full(first.size, i, dtype=np.int32), r0 + first,
                                       np.minimum(bq, n - first).astype(np.int32)], axis=1))
            arr = np.concatenate(parts).reshape(-1, 3) if parts else np.zeros((0, 3), dtype=np.int32)
            hit = (self._to_device(arr), int(arr.shape[0]))
            self._qblk[bq] = hit
        return hit
