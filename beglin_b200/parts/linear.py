"""y = x W^T (+ bias), W row-major [out, in] as in the checkpoint (qwen_infer.c:688-691).

float32: the hand-written CUDA-core kernel (true 32-bit, no tensor-core mode).
bfloat16: the tcgen05 tensor-core kernel of this package where it is the faster one (or everywhere,
with gemm="tcgen05"), else the vendor library's product, which is where the reference calls its own
platform's library (cblas_sgemv, qwen_infer.c:690).  Accumulation is float in every case.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from . import tensor_core
from .context import BuildContext


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor], ctx: BuildContext):
        self.ctx = ctx
        self.weight = ctx.matrix(weight)
        self.out_features, self.in_features = self.weight.shape
        self.bias_f32 = None if bias is None else bias.to(device=ctx.device, dtype=torch.float32).contiguous()
        self.bias_c = None if bias is None else self.bias_f32.to(ctx.compute_dtype)
        self.f32 = ctx.compute_dtype == torch.float32
        self._tc = None if self.f32 else tensor_core.plan(self.weight, ctx)
        self._tc_always = ctx.gemm == "tcgen05"

    def _run(self, x: torch.Tensor, out_dtype: torch.dtype, partial: bool) -> torch.Tensor:
        T = x.shape[0]
        if self.f32:
            out = torch.empty((T, self.out_features), dtype=torch.float32, device=x.device)
            ops.gemm_f32_nt(x, self.weight, self.bias_f32, out)
            return out
        if self._tc is not None and (self._tc_always or self._tc.wins(T)):
            return self._tc(x, self.bias_f32, out_dtype, partial)
        if out_dtype == torch.float32:
            y = torch.mm(x, self.weight.t(), out_dtype=torch.float32)
            if self.bias_f32 is not None:
                y += self.bias_f32
            return y
        if self.bias_c is not None:
            return torch.addmm(self.bias_c, x, self.weight.t())
        return torch.mm(x, self.weight.t())

    def __call__(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """x is [T, in] in the compute type; the result is [T, out] in `out_dtype` (default: compute type)."""
        return self._run(x, out_dtype or self.ctx.compute_dtype, False)

    def partial(self, x: torch.Tensor) -> torch.Tensor:
        """The product for a consumer kernel of this package (add_rmsnorm, swiglu, rope_kv_append), which
        takes either [T, out] or float partial sums [parts, T, out] over ranges of the inner size and
        adds them up itself."""
        return self._run(x, self.ctx.compute_dtype, True)
