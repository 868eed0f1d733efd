"""SwiGLU feed-forward: m = W_down (silu(W_gate h) * (W_up h)), no biases (qwen_infer.c:1560-1573,
:727-733).  Gate and up run as one product over the concatenated matrix [2*im, d], as the
reference fuses them (qwen_infer.c:1368-1402)."""
from __future__ import annotations

from typing import Dict, List

import torch

from ..csrc import ops
from .context import BuildContext
from .linear import Linear
from .registry import register_feed_forward
from .spec import SwiGLUSpec, TensorRole


@register_feed_forward("swiglu")
class SwiGLU:
    @staticmethod
    def expected_tensors(spec: SwiGLUSpec) -> List[TensorRole]:
        return [TensorRole("gate_proj.weight", (spec.intermediate, spec.hidden), True, True),
                TensorRole("up_proj.weight", (spec.intermediate, spec.hidden), True, True),
                TensorRole("down_proj.weight", (spec.hidden, spec.intermediate), True, True)]

    def __init__(self, spec: SwiGLUSpec, tensors: Dict[str, torch.Tensor], ctx: BuildContext):
        self.spec, self.ctx = spec, ctx
        self.gate_up = Linear(torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]], dim=0), None, ctx)
        self.down = Linear(tensors["down_proj.weight"], None, ctx)

    def forward(self, h: torch.Tensor, batch) -> torch.Tensor:
        gu = self.gate_up.partial(h)
        act = torch.empty((h.shape[0], self.spec.intermediate), dtype=self.ctx.compute_dtype, device=h.device)
        ops.swiglu(gu, act)
        return self.down.partial(act)
