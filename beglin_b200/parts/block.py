"""The arrangement of a layer's parts.  "prenorm" is the reference's decoder layer:
h = norm(x); x += mixer(h); h = norm(x); x += feed_forward(h)  (qwen_infer.c:1447, :1552, :1556,
:1577).  The residual x is float.  A block does not add its last result to x itself: it returns it,
and the next norm (of the next block, or the final one) adds it, fused with its statistics; or, in
steps of few tokens, the part's last product adds it and the next part's first product norms (see
stream.py)."""
from __future__ import annotations

from .registry import register_block
from .stream import NormedInput, ResidualStream


@register_block("prenorm")
class PreNormBlock:
    # the slots of a layer of this kind, in the order they are built: (slot name, family of the part).  A
    # block is constructed with one keyword argument per slot.
    SLOTS = (("mixer_norm", "norm"), ("mixer", "mixer"), ("feed_forward_norm", "norm"), ("feed_forward", "feed_forward"))

    def __init__(self, mixer_norm, mixer, feed_forward_norm, feed_forward):
        self.mixer_norm, self.mixer = mixer_norm, mixer
        self.feed_forward_norm, self.feed_forward = feed_forward_norm, feed_forward

    def forward(self, stream: ResidualStream, batch, cache) -> None:
        """Runs the layer on the residual stream.  A part that declares `takes_stream` gets the norm of the
        stream uncomputed (its first product may apply it) and the stream itself (its last product may add
        to it); any other part gets the normed rows and returns its addend, which the stream then owes."""
        h = NormedInput(stream, self.mixer_norm)
        if getattr(self.mixer, "takes_stream", False):
            a = self.mixer.forward(h, batch, cache, stream)
        else:
            a = self.mixer.forward(h.tensor(), batch, cache)
        if a is not None:
            stream.owe(a)
        h = NormedInput(stream, self.feed_forward_norm)
        if getattr(self.feed_forward, "takes_stream", False):
            m = self.feed_forward.forward(h, batch, stream)
        else:
            m = self.feed_forward.forward(h.tensor(), batch)
        if m is not None:
            stream.owe(m)
