"""Choosing the next token from a row of logits.

Greedy is the reference's only sampler: the index of the first maximum (qwen_infer.c:2152-2155).
Temperature sampling is added: p = softmax(logits / T) in float, inverted in index order at a
uniform number u.  u comes from a counter-based generator keyed by (seed, request, number of tokens
the request has generated), so a request's draws do not depend on what else is in its batch or on
how its steps were cut.  T = 0 means greedy.
"""
from __future__ import annotations

import zlib
from dataclasses import dataclass
from typing import Hashable, List, Sequence

import numpy as np
import torch

from ..csrc import ops

_MASK = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def request_key(rid: Hashable) -> int:
    if isinstance(rid, int) and not isinstance(rid, bool):
        return rid & _MASK
    return zlib.crc32(repr(rid).encode())


def uniform(seed: int, rid: Hashable, step: int) -> float:
    """A number in [0, 1) with 24 random bits, a pure function of its three arguments."""
    z = _splitmix64(seed & _MASK)
    z = _splitmix64(z ^ request_key(rid))
    z = _splitmix64(z ^ (step & _MASK))
    return (z >> 40) / float(1 << 24)


@dataclass
class SamplingParams:
    temperature: float = 0.0
    seed: int = 0


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, temperatures: Sequence[float], uniforms: Sequence[float]) -> List[int]:
        """One token per row of float logits [n, V]; rows with temperature <= 0 are greedy."""
        n = logits.shape[0]
        out = torch.empty(n, dtype=torch.int32, device=logits.device)
        if any(t > 0.0 for t in temperatures):
            t = torch.from_numpy(np.asarray(temperatures, dtype=np.float32)).to(logits.device)
            u = torch.from_numpy(np.asarray(uniforms, dtype=np.float32)).to(logits.device)
            ops.sample(logits, t, u, out)
        else:
            ops.sample(logits, None, None, out)
        return out.tolist()

    def greedy(self, logits: torch.Tensor) -> torch.Tensor:
        """Device int32 [n]: the first maximum of every row, without a host round trip."""
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
        ops.sample(logits, None, None, out)
        return out
