"""The float residual of a step and what is still owed to it.

A block's parts hand their results to the stream in one of two ways.  The plain way: the part
returns an addend (a tensor, or the partial sums of a split-K product) and the stream keeps it as
`pending` until the next norm adds it, fused with its statistics.  The fused way, for steps of few
tokens: the part's last product adds its result to `x` itself and leaves the sums of squares of the
new rows in `ssq`, and the next part's first product takes `x` and `ssq` and norms its operand on
the fly; then neither the addend nor the normed rows ever reach global memory, and two kernels of
the layer (the norms) and their launches are gone.
"""
from __future__ import annotations

from typing import Optional

import torch


class ResidualStream:
    def __init__(self, x: torch.Tensor):
        self.x = x                                     # float32 [T, d]
        self.pending: Optional[torch.Tensor] = None    # not yet added to x: [T, d] or partial sums [parts, T, d]
        self.ssq: Optional[torch.Tensor] = None        # float32 [parts, >= T]: partial sums of squares of x's rows

    def owe(self, addend: torch.Tensor) -> None:
        self.pending, self.ssq = addend, None

    def updated(self, ssq: Optional[torch.Tensor]) -> None:
        """x was changed in place by a fused product, which left these sums of squares."""
        self.pending, self.ssq = None, ssq


class NormedInput:
    """norm(stream) that has not been computed: a part whose first product can norm its operand takes
    it as it is (`Linear.of`); any other part asks for `tensor()`."""

    def __init__(self, stream: ResidualStream, norm):
        self.stream, self.norm = stream, norm
        self._tensor: Optional[torch.Tensor] = None

    @property
    def rows(self) -> int:
        return self.stream.x.shape[0]

    def tensor(self) -> torch.Tensor:
        if self._tensor is None:
            s = self.stream
            had = s.pending is not None
            self._tensor = self.norm.add_norm(s.x, s.pending)
            s.pending = None
            if had:
                s.ssq = None                            # x has changed
        return self._tensor

    def fusable(self):
        """(weight, eps) of the norm when a product may apply it to the stream itself, else None."""
        s = self.stream
        if self._tensor is not None or s.pending is not None or s.ssq is None:
            return None
        return getattr(self.norm, "fusion", lambda: None)()
