"""Choice of the tcgen05 tensor-core product for a weight matrix.  `plan` returns a callable
(x, bias, out_dtype) -> y for shapes the kernel takes, or None, in which case the caller uses the
vendor library's product."""
from __future__ import annotations

from typing import Callable, Optional

import torch

from .context import BuildContext


def plan(weight: torch.Tensor, ctx: BuildContext) -> Optional[Callable]:
    from ..csrc import ops
    maker = getattr(ops, "tcgen05_linear", None)
    if maker is None:
        if ctx.gemm == "tcgen05":
            raise RuntimeError("the tcgen05 product was asked for but the kernel library does not have it")
        return None
    return maker(weight, required=(ctx.gemm == "tcgen05"))
