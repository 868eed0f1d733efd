"""Descriptions of the parts a model is put together from.  Pure data: no tensors, no device.

A model is a `ModelSpec`: an embedding, a list of layers, the order in which the layers run, a
final norm and a head.  Every layer names the kind of its block, mixer, feed-forward, norms and
position encoding and gives each its sizes and constants, so two layers of one model may differ in
all of them.  The kinds are looked up in the registries of `beglin_b200.parts.registry`; a spec
never names the architecture it came from.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


@dataclass(frozen=True)
class TensorRole:
    """One tensor a part wants: its name inside the part, its shape, whether it may be absent,
    whether it is a matrix of a matrix product (kept in the compute dtype) or a small vector or
    table (kept as stored), and what it is for.  `role` decides how random weights are drawn:
    "matrix" and "vector" around zero, "bias" around zero with a deviation of its own, "scale" (a
    norm's weight, which multiplies) around one.  Empty means "matrix" or "vector" by `matrix`."""
    name: str
    shape: Tuple[int, ...]
    required: bool = True
    matrix: bool = False
    role: str = ""

    def init_role(self) -> str:
        return self.role or ("matrix" if self.matrix else "vector")


@dataclass(frozen=True)
class NormSpec:
    size: int
    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class PositionSpec:
    """Rotary position encoding: `rotary_dim` leading features of each head are rotated in pairs,
    (i, i + rotary_dim/2) for pairing "split_half" (qwen_infer.c:782-790) or (2i, 2i+1) for
    "interleaved" (qwen_infer.c:738-750); frequency i is theta^(-2i/rotary_dim) * freq_scale[i]
    (qwen_infer.c:757-794).  kind "none" rotates nothing."""
    kind: str = "rope"
    rotary_dim: int = 0
    theta: float = 10000.0
    pairing: str = "split_half"
    freq_scale: Optional[Tuple[float, ...]] = None


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query attention over a paged cache.  `window` None means all earlier positions; a
    number w means the last w positions, the token itself included.  `own_kv` False makes a mixer
    that projects no keys and values of its own and reads the cache of another stage."""
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    qkv_bias: bool
    position: PositionSpec
    out_bias: bool = False
    window: Optional[int] = None
    scale: Optional[float] = None          # None: 1/sqrt(head_dim)  (qwen_infer.c:1488)
    own_kv: bool = True
    kind: str = "gqa_attention"


@dataclass(frozen=True)
class SwiGLUSpec:
    hidden: int
    intermediate: int
    kind: str = "swiglu"


class LayerSpec:
    """One decoder layer: the kind of its block, and the spec of the part in every slot that the block
    kind declares (`parts`: slot name -> part spec; the block class's `SLOTS` says which slots there are
    and of which family each is).  `names` maps each part's own tensor names, qualified by the slot, to
    checkpoint names, e.g. {"mixer.q_proj.weight": "model.layers.3.self_attn.q_proj.weight"}.

    The slots may also be given as keywords (`LayerSpec(mixer=..., feed_forward=..., names=...)`) and
    read as attributes (`layer.mixer`); `with_parts` returns a copy with some slots, the names or the
    block kind replaced."""

    def __init__(self, parts: Optional[Dict[str, object]] = None, names: Optional[Dict[str, str]] = None,
                 block: str = "prenorm", **slots):
        merged = dict(parts or {})
        merged.update(slots)
        object.__setattr__(self, "parts", merged)
        object.__setattr__(self, "names", dict(names or {}))
        object.__setattr__(self, "block", block)

    def __getattr__(self, slot):
        parts = self.__dict__.get("parts", {})
        if slot in parts:
            return parts[slot]
        raise AttributeError(f"the layer has no slot '{slot}' (slots: {', '.join(parts) or 'none'})")

    def __setattr__(self, key, value):
        raise AttributeError("a LayerSpec is not changed in place; use with_parts()")

    def with_parts(self, names: Optional[Dict[str, str]] = None, block: Optional[str] = None, **slots) -> "LayerSpec":
        parts = dict(self.parts)
        parts.update(slots)
        return LayerSpec(parts, self.names if names is None else names, self.block if block is None else block)

    def __repr__(self):
        return f"LayerSpec(block={self.block!r}, parts={self.parts!r})"


@dataclass(frozen=True)
class Stage:
    """One entry of the run order: which layer runs, and whose cache it uses.  `cache` None means
    a cache of its own; a number names an earlier stage of the order whose cache is read."""
    layer: int
    cache: Optional[int] = None


@dataclass
class ModelSpec:
    vocab: int
    hidden: int
    layers: List[LayerSpec]
    order: List[Stage]
    final_norm: NormSpec
    embed_name: str
    final_norm_name: str
    head_name: Optional[str]              # None: the head is the embedding table (tied)
    max_positions: Optional[int] = None
    embed_scale: float = 1.0              # the embedded rows are multiplied by this (1: as they are)
    head_bias_name: Optional[str] = None  # a bias [vocab] added to the logits
    logit_softcap: float = 0.0            # c > 0: logits = c * tanh(logits / c)
    eos_ids: Tuple[int, ...] = ()
    extra: Dict[str, object] = field(default_factory=dict)
