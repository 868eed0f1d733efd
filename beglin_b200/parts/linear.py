"""y = x W^T (+ bias), W row-major [out, in] as in the checkpoint (qwen_infer.c:688-691).

float32: the hand-written CUDA-core kernel (true 32-bit, no tensor-core mode).
bfloat16: the tcgen05 tensor-core kernel of this package where it is the faster one (or everywhere,
with gemm="tcgen05"), else the vendor library's product, which is where the reference calls its own
platform's library (cblas_sgemv, qwen_infer.c:690).  Accumulation is float in every case: the library
is told not to add up in bfloat16 the parts of a product that it splits along the inner size, which it
otherwise does for few rows (measured on a tiny model: the error of eight decoded rows 0.015 against 0.008
of the same rows one by one).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from . import tensor_core
from .context import BuildContext
from .stream import NormedInput, ResidualStream


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor], ctx: BuildContext, label: str = "proj"):
        """`label` names the product's kernel class for the phase timers (ops.phase)."""
        self.ctx = ctx
        self.label = label
        self.weight = ctx.matrix(weight)
        self.out_features, self.in_features = self.weight.shape
        self.bias_f32 = None if bias is None else bias.to(device=ctx.device, dtype=torch.float32).contiguous()
        self.bias_c = None if bias is None else self.bias_f32.to(ctx.compute_dtype)
        self.f32 = ctx.compute_dtype == torch.float32
        self._tc = None if self.f32 else tensor_core.plan(self.weight, ctx)
        self._tc_always = ctx.gemm == "tcgen05"
        if not self.f32:
            torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False

    def _run(self, x: torch.Tensor, out_dtype: torch.dtype, partial: bool) -> torch.Tensor:
        with ops.phase(self.label):
            return self._product(x, out_dtype, partial)

    def _product(self, x: torch.Tensor, out_dtype: torch.dtype, partial: bool) -> torch.Tensor:
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

    # ------------------------------------------------------------------ products that take over their neighbours' work
    def fuses(self, T: int) -> bool:
        """Whether a step of T rows runs the fused product (bfloat16, few tokens, sizes it takes)."""
        return self._tc is not None and self._tc.fuses(T)

    def _check_rows(self, x: torch.Tensor) -> None:
        if x.dtype != torch.bfloat16 or x.stride(1) != 1 or x.shape[1] != self.in_features or x.stride(0) % 8:
            raise ops.KernelError(f"the fused product takes contiguous bfloat16 rows of {self.in_features} features")

    def of(self, inp, swiglu: bool = False) -> torch.Tensor:
        """The product of `inp`, a tensor [T, in] or a NormedInput (a norm of the residual stream that has
        not been computed).  Where the fused product runs, the norm is applied to the operand inside it;
        the result is then complete ([T, out], float).  Else as `partial`.  With `swiglu` (the weight's
        rows interleaved in blocks of 64, gate then up) the result is silu(gate) * up, [T, out / 2] in the
        compute type (from the fused product of few rows or from the product of many rows on pairs of CTAs), or
        None when this step runs neither."""
        lazy = isinstance(inp, NormedInput)
        T = inp.rows if lazy else inp.shape[0]
        if not self.fuses(T):
            if swiglu:
                if self._tc is None or not self._tc.pairs(T):
                    return None
                with ops.phase(self.label):
                    return self._tc.pair_swiglu(inp.tensor() if lazy else inp)
            return self.partial(inp.tensor() if lazy else inp)
        fusion = inp.fusable() if lazy else None
        n = self.out_features // 2 if swiglu else self.out_features
        out = torch.empty((T, n), dtype=self.ctx.compute_dtype if swiglu else torch.float32, device=self.weight.device)
        mode = ops.FUSED_SWIGLU if swiglu else ops.FUSED_PLAIN
        if fusion is not None:
            weight, eps = fusion
            with ops.phase(self.label):
                self._tc.fused(T, out, mode, xf=inp.stream.x, ssq_in=inp.stream.ssq, norm_weight=weight, eps=eps,
                               bias=self.bias_f32)
        else:
            x = inp.tensor() if lazy else inp
            self._check_rows(x)
            with ops.phase(self.label):
                self._tc.fused(T, out, mode, x=x, bias=self.bias_f32)
        return out

    def rope_fuses(self, T: int, hd: int) -> bool:
        """Whether a step of T rows runs this (q/k/v) product with rotation and cache append inside it: where the
        fused product runs, the heads fit its tiles, and the product has CTAs for at least half of the SMs (measured
        in one run each: 1.283 against 1.354 ms a step at the 1.5B sizes with 128 CTAs and 3.69 against 3.71 ms at
        the 7B sizes with 144, but 0.954 against 0.943 ms at the 0.5B sizes, whose 36 CTAs take 2 us longer for
        it, as long as the kernel that it saves).  A context built with fuse="all" fuses whatever the sizes allow."""
        if not self.fuses(T) or hd not in self._tc.ROPE_HEAD_SIZES:
            return False
        return self.ctx.fuse == "all" or 2 * self._tc.tiles * self._tc.fused_splits(T) >= self._tc.sms

    def of_rope(self, inp, q_out: torch.Tensor, rope: tuple) -> None:
        """The q/k/v product of `inp` (as `of`) with the rotation of queries and keys and the append of keys and
        values to the cache inside it: q_out [T, nh hd] receives the queries; `rope` is (cos_sin, positions,
        row_req, block_table, kv_pool, page_size, nh, nkv, hd).  Only where `rope_fuses`."""
        lazy = isinstance(inp, NormedInput)
        T = inp.rows if lazy else inp.shape[0]
        fusion = inp.fusable() if lazy else None
        with ops.phase(self.label):
            if fusion is not None:
                weight, eps = fusion
                self._tc.fused_rope(T, q_out, rope, xf=inp.stream.x, ssq_in=inp.stream.ssq, norm_weight=weight, eps=eps,
                                    bias=self.bias_f32)
            else:
                x = inp.tensor() if lazy else inp
                self._check_rows(x)
                self._tc.fused_rope(T, q_out, rope, x=x, bias=self.bias_f32)

    def into(self, x: torch.Tensor, stream: ResidualStream) -> None:
        """stream += x W^T (+ bias).  Where the fused product runs it adds to the stream itself and leaves
        the sums of squares of the new rows for the next norm; else the result is owed to the stream."""
        T = x.shape[0]
        if self.fuses(T) and stream.pending is None:
            self._check_rows(x)
            with ops.phase(self.label):
                stream.updated(self._tc.fused(T, stream.x, ops.FUSED_RESIDUAL, x=x, bias=self.bias_f32, want_ssq=True))
        elif self._tc_always and T >= tensor_core.PAIR_TOKENS and stream.pending is None and self.out_features % 4 == 0:
            with ops.phase(self.label):
                self._tc.pair_residual(x, self.bias_f32, stream.x)
            stream.updated(None)
        else:
            stream.owe(self.partial(x))
