"""The arrangement of a layer's parts.  "prenorm" is the reference's decoder layer:
h = norm(x); x += mixer(h); h = norm(x); x += feed_forward(h)  (qwen_infer.c:1447, :1552, :1556,
:1577).  The residual x is float.  A block does not add its last result to x itself: it returns it,
and the next norm (of the next block, or the final one) adds it, fused with its statistics."""
from __future__ import annotations

from typing import Optional

import torch

from .registry import register_block


@register_block("prenorm")
class PreNormBlock:
    def __init__(self, mixer_norm, mixer, feed_forward_norm, feed_forward):
        self.mixer_norm, self.mixer = mixer_norm, mixer
        self.feed_forward_norm, self.feed_forward = feed_forward_norm, feed_forward

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], batch, cache) -> torch.Tensor:
        """x: float residual [T, d], to which `pending` has not been added yet.  Returns the new
        pending addend."""
        h = self.mixer_norm.add_norm(x, pending)
        a = self.mixer.forward(h, batch, cache)
        h = self.feed_forward_norm.add_norm(x, a)
        return self.feed_forward.forward(h, batch)
