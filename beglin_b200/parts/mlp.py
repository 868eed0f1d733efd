"""SwiGLU feed-forward: m = W_down (silu(W_gate h) * (W_up h)), no biases (qwen_infer.c:1560-1573,
:727-733).  Gate and up run as one product over the concatenated matrix [2*im, d], as the
reference fuses them (qwen_infer.c:1368-1402)."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..csrc import ops
from .context import BuildContext
from .linear import Linear
from .registry import register_feed_forward
from .spec import SwiGLUSpec, TensorRole
from .stream import ResidualStream


@register_feed_forward("swiglu")
class SwiGLU:
    @staticmethod
    def expected_tensors(spec: SwiGLUSpec) -> List[TensorRole]:
        return [TensorRole("gate_proj.weight", (spec.intermediate, spec.hidden), True, True),
                TensorRole("up_proj.weight", (spec.intermediate, spec.hidden), True, True),
                TensorRole("down_proj.weight", (spec.hidden, spec.intermediate), True, True)]

    takes_stream = True        # forward takes a NormedInput and may add its result to the stream itself

    def __init__(self, spec: SwiGLUSpec, tensors: Dict[str, torch.Tensor], ctx: BuildContext):
        self.spec, self.ctx = spec, ctx
        gate, up, im = tensors["gate_proj.weight"], tensors["up_proj.weight"], spec.intermediate
        # Where the intermediate size allows it, the rows go in blocks of 64: gate, up, gate, up, ...  A CTA of
        # the fused product (128 rows) then holds 64 gate features with their 64 up features and applies
        # silu(gate) * up itself; the plain kernel reads the same layout.
        self.block = 64 if im % 64 == 0 else 0
        if self.block:
            w = torch.stack([gate.reshape(im // 64, 64, -1), up.reshape(im // 64, 64, -1)], dim=1).reshape(2 * im, -1)
        else:
            w = torch.cat([gate, up], dim=0)
        self.gate_up = Linear(w, None, ctx, label="proj_gate_up")
        self.down = Linear(tensors["down_proj.weight"], None, ctx, label="proj_down")

    def forward(self, h, batch, stream: Optional[ResidualStream] = None) -> Optional[torch.Tensor]:
        """h: the normed rows, or a NormedInput.  With `stream` the result is added to it (or left owed to
        it) and None is returned; without, the addend is returned."""
        act = self.gate_up.of(h, swiglu=True) if self.block else None
        if act is None:
            gu = self.gate_up.of(h)
            act = torch.empty((gu.shape[-2], self.spec.intermediate), dtype=self.ctx.compute_dtype, device=gu.device)
            ops.swiglu(gu, act, self.block)
        if stream is None:
            return self.down.partial(act)
        self.down.into(act, stream)
        return None
