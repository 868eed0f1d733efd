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
