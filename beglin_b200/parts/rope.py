"""Rotary position encoding.  Frequency i is theta^(-2i/rot) * scale_i; the angle of a token is its
position times the frequency, as a float product, and its cosine and sine are computed once per
step for all layers and heads (qwen_infer.c:757-794).  The table is made by the `rope_table`
kernel; the rotation itself is fused into the cache append (`rope_kv_append`).

The frequencies are 32-bit numbers made the way the reference makes them (qwen_infer.c:791):
`powf(theta, -(2.0f*i)/hd)` of the 32-bit theta and the 32-bit exponent, times the 32-bit scale.
`powf` is taken as correctly rounded (the power in 64-bit of the 32-bit operands, rounded once), so
that the same bits come out on every host; at position 30,000 one unit in a frequency's last place
moves the angle by 0.002."""
from __future__ import annotations

import numpy as np
import torch

from ..csrc import ops
from .context import BuildContext
from .registry import register_position
from .spec import PositionSpec


@register_position("rope")
class RotaryPosition:
    def __init__(self, spec: PositionSpec, ctx: BuildContext):
        if spec.rotary_dim <= 0 or spec.rotary_dim % 2:
            raise ValueError(f"rotary_dim={spec.rotary_dim} must be positive and even")
        if spec.pairing not in ("split_half", "interleaved"):
            raise ValueError(f"unknown rotary pairing '{spec.pairing}'")
        self.spec, self.ctx = spec, ctx
        half = spec.rotary_dim // 2
        exponent = -(np.float32(2.0) * np.arange(half, dtype=np.float32)) / np.float32(spec.rotary_dim)
        inv = np.power(np.float64(np.float32(spec.theta)), exponent.astype(np.float64)).astype(np.float32)
        if spec.freq_scale is not None:
            if len(spec.freq_scale) != half:
                raise ValueError("freq_scale must have rotary_dim/2 entries")
            inv = inv * np.asarray(spec.freq_scale, dtype=np.float32)
        self.inv_freq = torch.from_numpy(inv.astype(np.float32)).to(ctx.device)
        self.rotary_dim = spec.rotary_dim
        self.interleaved = spec.pairing == "interleaved"

    def table(self, batch) -> torch.Tensor:
        """float32 [T, rot/2, 2] of (cos, sin) for the step's rows; made once per step."""
        key = ("rope_table", id(self))
        t = batch.scratch.get(key)
        if t is None:
            t = torch.empty((batch.n_rows, self.rotary_dim // 2, 2), dtype=torch.float32, device=self.ctx.device)
            ops.rope_table(batch.positions, self.inv_freq, t)
            batch.scratch[key] = t
        return t


@register_position("none")
class NoPosition:
    def __init__(self, spec: PositionSpec, ctx: BuildContext):
        self.spec, self.ctx = spec, ctx
        self.rotary_dim = 0
        self.interleaved = False

    def table(self, batch):
        return None


def shared_position(spec: PositionSpec, ctx: BuildContext):
    """One part per distinct spec, so layers with the same encoding share one table per step."""
    from .registry import position_class
    key = ("position", spec)
    part = ctx.shared.get(key)
    if part is None:
        part = position_class(spec.kind)(spec, ctx)
        ctx.shared[key] = part
    return part
