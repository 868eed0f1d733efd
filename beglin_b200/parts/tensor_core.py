"""Choice between the tcgen05 tensor-core product of this package and the vendor library's product
for a bfloat16 weight matrix, and the split of K for steps of few tokens.

With few tokens a product is bound by streaming the weight matrix once, and a matrix with few
128-row tiles would leave most SMs idle; K is then cut into ranges, each CTA writes a float partial
sum, and the kernel that consumes the result adds the partial sums in index order.  How many ranges
depends only on the matrix's shape and the number of tokens in the step.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from .context import BuildContext

FEW_TOKENS = 64            # up to this many rows a product is treated as weight-streaming
FUSED_TOKENS = 16            # steps of up to this many rows run the fused product (measured: it loses from 32 rows on)
PAIR_TOKENS = 192            # from this many rows on the product with SwiGLU in its epilogue runs on pairs of CTAs


class TensorCoreProduct:
    def __init__(self, weight: torch.Tensor, ctx: BuildContext):
        self.weight, self.ctx = weight, ctx
        self.n_out, self.k = weight.shape
        self.tiles = -(-self.n_out // 128)
        self.k_blocks = -(-self.k // 64)
        ops.lib()
        self._w_ptr, self._ldw = weight.data_ptr(), weight.stride(0)
        self._status_ptr = None if ctx.status is None else ctx.status.data_ptr()
        self._splits = {}
        self.sms = ops.sm_count(weight.device)

    @staticmethod
    def takes(weight: torch.Tensor) -> bool:
        return weight.dtype == torch.bfloat16 and weight.shape[1] % 8 == 0 and weight.stride(0) % 8 == 0

    def wins(self, T: int) -> bool:
        """Whether this kernel is the faster one for a step of T rows (measured on B200 at the
        Qwen2.5-1.5B shapes): it is for few tokens, where the product is a stream of weights, K is
        cut so that every SM has work, and under programmatic dependent launch the weight tiles are
        requested while the previous kernel still runs, which the library's kernel cannot do."""
        return T <= FEW_TOKENS

    def splits(self, T: int) -> int:
        s = self._splits.get(T)
        if s is None:
            s = self._splits[T] = self._choose_splits(T)
        return s

    def _choose_splits(self, T: int) -> int:
        if T > FEW_TOKENS:
            return 1
        want = max(1, -(-self.sms // self.tiles))                 # enough CTAs for every SM
        want = min(want, max(1, self.k_blocks // 2))              # at least two k-blocks per range
        want = min(want, max(1, self.k // (8 * T)))               # partial sums stay a fraction of the weight bytes
        per = -(-self.k_blocks // want)
        return -(-self.k_blocks // per)                           # no empty range

    # ------------------------------------------------------------------ the fused product of few-token steps
    def fuses(self, T: int) -> bool:
        return self.ctx.fuse and T <= FUSED_TOKENS and self.k % 8 == 0

    def fused_splits(self, T: int) -> int:
        """1, 2, 4, 8 or 16 ranges of K (the CTAs of a tile form a cluster): enough CTAs for every SM, at
        least two k-blocks per range, no empty range."""
        s = self._splits.get(("fused", T))
        if s is None:
            want = max(1, -(-self.sms // (self.tiles * -(-T // 64))))
            s = 1
            while s < 16 and s < want and 2 * s <= max(1, self.k_blocks // 2):
                s *= 2
            while s > 1 and (s - 1) * -(-self.k_blocks // s) >= self.k_blocks:
                s //= 2
            self._splits[("fused", T)] = s
        return s

    def fused(self, T: int, out: torch.Tensor, mode: int, x: Optional[torch.Tensor] = None,
              xf: Optional[torch.Tensor] = None, ssq_in: Optional[torch.Tensor] = None,
              norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0, bias: Optional[torch.Tensor] = None,
              want_ssq: bool = False) -> Optional[torch.Tensor]:
        """ops.gemm_fused with this weight; returns the sums of squares of the new rows when asked."""
        s = self.fused_splits(T)
        ssq_out = torch.empty((self.tiles * s, 64), dtype=torch.float32, device=out.device) if want_ssq else None
        ops.gemm_fused_unchecked(self._w_ptr, self.n_out, self.k, self._ldw, T, out, mode, x, xf, ssq_in,
                                 None if norm_weight is None else norm_weight.data_ptr(), eps,
                                 None if bias is None else bias.data_ptr(), ssq_out, s, self._status_ptr)
        return ssq_out

    ROPE_HEAD_SIZES = (32, 64, 128)      # whole heads in a tile of 128 rows, so that a feature meets its partner

    def fused_rope(self, T: int, q_out: torch.Tensor, rope: tuple, x: Optional[torch.Tensor] = None,
                   xf: Optional[torch.Tensor] = None, ssq_in: Optional[torch.Tensor] = None,
                   norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0, bias: Optional[torch.Tensor] = None) -> None:
        """The q/k/v product with rotation and cache append behind it; `rope` is (cos_sin, positions, row_req,
        block_table, kv_pool, page_size, nh, nkv, hd)."""
        ops.gemm_fused_rope_unchecked(self._w_ptr, self.k, self._ldw, T, q_out, x, xf, ssq_in,
                                      None if norm_weight is None else norm_weight.data_ptr(), eps,
                                      None if bias is None else bias.data_ptr(), *rope, self.fused_splits(T), self._status_ptr)

    # ------------------------------------------------------------------ the product of many rows on pairs of CTAs
    def pairs(self, T: int) -> bool:
        """Whether a step of T rows runs gate/up with SwiGLU as ONE kernel of CTA pairs (measured at the 1.5B and
        7B shapes: from 256 rows on it beats the library's product followed by the SwiGLU kernel by 10 to 25 %;
        at 128 rows it loses by 6 %).  The plain products of many rows stay with the library: their matrices
        have too few 256 x 256 tiles for the pairs of the device."""
        return self.ctx.fuse and T >= PAIR_TOKENS and self.n_out % 128 == 0

    def pair_swiglu(self, x: torch.Tensor) -> torch.Tensor:
        """silu(gate) * up of x's rows, [T, n_out / 2] bfloat16; the weight's rows are interleaved in blocks of 64."""
        if x.dtype != torch.bfloat16 or x.stride(1) != 1 or x.shape[1] != self.k or x.stride(0) % 8:
            raise ops.KernelError(f"the tcgen05 product takes contiguous bfloat16 rows of {self.k} features")
        out = torch.empty((x.shape[0], self.n_out // 2), dtype=torch.bfloat16, device=x.device)
        ops.gemm_pair_unchecked(x, self._w_ptr, self.n_out, self.k, self._ldw, out, ops.PAIR_SWIGLU, self._status_ptr)
        return out

    def pair_residual(self, x: torch.Tensor, bias: Optional[torch.Tensor], stream_x: torch.Tensor) -> None:
        """stream_x (float32 [T, n_out]) += x W^T (+ bias) on pairs of CTAs.  Measured slower than the library's
        product followed by the add-and-norm kernel at the 1.5B and 7B shapes (58 against 50 us for the down
        product of 2,048 tokens), so only an engine built with gemm="tcgen05" runs it."""
        if x.dtype != torch.bfloat16 or x.stride(1) != 1 or x.shape[1] != self.k or x.stride(0) % 8:
            raise ops.KernelError(f"the tcgen05 product takes contiguous bfloat16 rows of {self.k} features")
        ops.gemm_pair_unchecked(x, self._w_ptr, self.n_out, self.k, self._ldw, stream_x, ops.PAIR_RESIDUAL,
                                self._status_ptr, None if bias is None else bias.data_ptr())

    def __call__(self, x: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype, partial: bool) -> torch.Tensor:
        T = x.shape[0]
        if T >= PAIR_TOKENS and out_dtype == torch.bfloat16:
            # many rows (this kernel is asked for them only by an engine built with gemm="tcgen05"): pairs of CTAs
            if x.dtype != torch.bfloat16 or x.stride(1) != 1 or x.shape[1] != self.k or x.stride(0) % 8:
                raise ops.KernelError(f"the tcgen05 product takes contiguous bfloat16 rows of {self.k} features")
            out = torch.empty((T, self.n_out), dtype=torch.bfloat16, device=x.device)
            ops.gemm_pair_unchecked(x, self._w_ptr, self.n_out, self.k, self._ldw, out, ops.PAIR_PLAIN, self._status_ptr,
                                    None if bias is None else bias.data_ptr())
            return out
        s = self.splits(T) if partial else 1
        if s > 1:
            out = torch.empty((s, T, self.n_out), dtype=torch.float32, device=x.device)
        else:
            out = torch.empty((T, self.n_out), dtype=out_dtype, device=x.device)
        if x.dtype != torch.bfloat16 or x.stride(1) != 1 or x.shape[1] != self.k or x.stride(0) % 8:
            raise ops.KernelError(f"the tcgen05 product takes contiguous bfloat16 rows of {self.k} features")
        ops.gemm_bf16_tn_unchecked(x, self._w_ptr, self.n_out, self.k, self._ldw, None if bias is None else bias.data_ptr(),
                                   out, s, self._status_ptr)
        return out


def plan(weight: torch.Tensor, ctx: BuildContext) -> Optional[TensorCoreProduct]:
    if ctx.gemm == "library":
        return None
    if not TensorCoreProduct.takes(weight):
        if ctx.gemm == "tcgen05":
            raise ValueError(f"the tcgen05 product was asked for, but it does not take a {tuple(weight.shape)} "
                             f"{weight.dtype} matrix (bfloat16, inner size a multiple of 8)")
        return None
    return TensorCoreProduct(weight, ctx)
