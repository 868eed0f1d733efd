"""What every part is built with: the device, the compute and cache types, and the status word of
the kernels.  A part gets its sizes from its spec and everything about the machine from here."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional

import torch


@dataclass
class BuildContext:
    device: torch.device
    compute_dtype: torch.dtype              # torch.float32 (true 32-bit path) or torch.bfloat16
    cache_dtype: Optional[torch.dtype] = None
    page_size: int = 64
    # keys per split of the CUDA-core attention (the float32 path and odd sizes): fixed positions, so a row's result
    # does not depend on the batch.  The bfloat16 decoding kernel spreads a request's keys over its CTAs by the
    # step's shapes instead: its rows agree between batches to rounding, not bit for bit.
    kv_split: int = 256
    gemm: str = "auto"                      # "auto", "library" or "tcgen05" for the bfloat16 products
    attention: str = "auto"                 # "auto", "generic" (CUDA cores) or "mma" (tensor cores) kernel
    # few-token steps: norms, residual adds, SwiGLU, rotation and cache append inside the products.  True: where it was
    # measured to pay; "all": wherever the sizes allow it (tests of the fused kernels on tiny models); False: nowhere
    fuse: object = True
    status: Optional[torch.Tensor] = None   # device word in which kernels record bad ids and pages
    shared: Dict[object, object] = field(default_factory=dict)   # parts shared between layers, by spec

    def __post_init__(self):
        self.device = torch.device(self.device)
        if self.compute_dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype must be float32 or bfloat16, got {self.compute_dtype}")
        if self.cache_dtype is None:
            self.cache_dtype = self.compute_dtype
        if self.kv_split % 64 != 0:
            raise ValueError("kv_split must be a multiple of 64")

    def matrix(self, t: torch.Tensor) -> torch.Tensor:
        """A matrix of a matrix product: on the device, in the compute type."""
        return t.to(device=self.device, dtype=self.compute_dtype).contiguous()

    def vector(self, t: torch.Tensor) -> torch.Tensor:
        """A small vector (norm weight, bias): on the device, float32 stays float32, everything else
        becomes the compute type."""
        dt = torch.float32 if t.dtype == torch.float32 else self.compute_dtype
        return t.to(device=self.device, dtype=dt).contiguous()
