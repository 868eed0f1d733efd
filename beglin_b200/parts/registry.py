"""Registries from the `kind` of a spec to the class that runs it.

A part is registered under the kind its spec carries; `build_*` looks the kind up and constructs the
part from (spec, tensors, context).  Code outside the package may register further kinds (tests
register toy mixers this way), so adding a part changes no file of the framework.
"""
from __future__ import annotations

from typing import Callable, Dict

MIXERS: Dict[str, type] = {}
FEED_FORWARDS: Dict[str, type] = {}
NORMS: Dict[str, type] = {}
POSITIONS: Dict[str, type] = {}
BLOCKS: Dict[str, type] = {}


def _register(table: Dict[str, type], what: str) -> Callable[[str], Callable[[type], type]]:
    def by_kind(kind: str):
        def deco(cls: type) -> type:
            table[kind] = cls
            cls.kind = kind
            return cls
        return deco
    return by_kind


register_mixer = _register(MIXERS, "mixer")
register_feed_forward = _register(FEED_FORWARDS, "feed-forward")
register_norm = _register(NORMS, "norm")
register_position = _register(POSITIONS, "position encoding")
register_block = _register(BLOCKS, "block")


def lookup(table: Dict[str, type], kind: str, what: str) -> type:
    try:
        return table[kind]
    except KeyError:
        known = ", ".join(sorted(table)) or "(none)"
        raise KeyError(f"no {what} of kind '{kind}' is registered; registered: {known}") from None


def mixer_class(kind: str) -> type:
    return lookup(MIXERS, kind, "mixer")


def feed_forward_class(kind: str) -> type:
    return lookup(FEED_FORWARDS, kind, "feed-forward")


def norm_class(kind: str) -> type:
    return lookup(NORMS, kind, "norm")


def position_class(kind: str) -> type:
    return lookup(POSITIONS, kind, "position encoding")


def block_class(kind: str) -> type:
    return lookup(BLOCKS, kind, "block")


FAMILIES = {"mixer": (MIXERS, "mixer"), "feed_forward": (FEED_FORWARDS, "feed-forward"), "norm": (NORMS, "norm")}


def part_class(family: str, kind: str) -> type:
    """The class of a part of one of the families a block's slots are made of."""
    try:
        table, what = FAMILIES[family]
    except KeyError:
        raise KeyError(f"no family of parts called '{family}'; families: {', '.join(FAMILIES)}") from None
    return lookup(table, kind, what)


def layer_slots(layer) -> list:
    """(slot name, family, part class, part spec) for every slot that the layer's block kind declares,
    in the block's order.  A slot the layer's spec does not fill, or a part the block has no slot for,
    is an error."""
    block = block_class(layer.block)
    slots = getattr(block, "SLOTS", None)
    if slots is None:
        raise TypeError(f"block kind '{layer.block}' declares no SLOTS")
    declared = [name for name, _ in slots]
    missing = [name for name in declared if name not in layer.parts]
    extra = [name for name in layer.parts if name not in declared]
    if missing or extra:
        raise KeyError(f"a layer of block kind '{layer.block}' has slots {declared}; "
                       f"the spec lacks {missing} and has {extra} besides")
    if sum(1 for _, family in slots if family == "mixer") > 1:
        raise TypeError(f"block kind '{layer.block}' declares more than one mixer slot; a stage has one cache")
    return [(name, family, part_class(family, layer.parts[name].kind), layer.parts[name]) for name, family in slots]
