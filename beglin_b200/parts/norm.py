"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * weight, statistics in float, eps inside the root, the
weight multiplying directly (qwen_infer.c:711-714).  The residual add that precedes a norm is fused
into it: `add_norm` first does x += delta."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..csrc import ops
from .context import BuildContext
from .registry import register_norm
from .spec import NormSpec, TensorRole


@register_norm("rmsnorm")
class RMSNorm:
    @staticmethod
    def expected_tensors(spec: NormSpec) -> List[TensorRole]:
        return [TensorRole("weight", (spec.size,), role="scale")]

    def __init__(self, spec: NormSpec, tensors: Dict[str, torch.Tensor], ctx: BuildContext):
        self.spec, self.ctx = spec, ctx
        self.weight = ctx.vector(tensors["weight"])

    def add_norm(self, x: torch.Tensor, delta: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None,
                 update: bool = True) -> torch.Tensor:
        """x is the float residual [T, size].  x += delta (when given and `update`), then the normed
        rows in the compute type.  With `rows`, only those rows are normed and x is left alone."""
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.spec.size), dtype=self.ctx.compute_dtype, device=x.device)
        ops.add_rmsnorm(x, delta, self.weight, self.spec.eps, out, rows=rows, update=update and rows is None)
        return out

    def fusion(self):
        """What a product needs to apply this norm to its operand itself: (weight, eps); None when the
        weight is not in the compute type (a checkpoint that stores it in 32-bit keeps it so)."""
        if self.weight.dtype != self.ctx.compute_dtype:
            return None
        return self.weight, float(self.spec.eps)
