"""Binding a model's parts to checkpoint tensors by name.

`expected_tensors(spec)` asks every part of a `ModelSpec` which tensors it wants (name inside the
part, shape, required or optional) and translates the names through the layer's name map into
checkpoint names.  `bind` compares that list with what a checkpoint holds and raises ONE
`WeightError` that lists the missing tensors, the unexpected ones and those of a wrong shape.  The
reference stops at the first missing name (qwen_infer.c:19501) and trusts the stored shapes
(:19516-19517); checking the shapes against the configuration is added here.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from ..parts import registry
from ..parts.spec import ModelSpec, TensorRole


class WeightError(ValueError):
    def __init__(self, missing, unexpected, wrong_shape, origin=""):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        lines = [f"weights do not fit the model{' (' + origin + ')' if origin else ''}:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        super().__init__("\n".join(lines))


def layer_roles(layer) -> List[Tuple[str, TensorRole]]:
    """(slot-qualified name, role) of every tensor a layer's parts want: the slots are those its block
    kind declares."""
    out: List[Tuple[str, TensorRole]] = []
    for slot, _, cls, spec in registry.layer_slots(layer):
        for role in cls.expected_tensors(spec):
            out.append((f"{slot}.{role.name}", role))
    return out


def expected_tensors(spec: ModelSpec) -> Dict[str, TensorRole]:
    """Checkpoint name -> role (shape, required, matrix) for the whole model."""
    import beglin_b200.parts  # noqa: F401  (registers the built-in parts)
    out: Dict[str, TensorRole] = {}
    out[spec.embed_name] = TensorRole(spec.embed_name, (spec.vocab, spec.hidden), True, True)
    for li, layer in enumerate(spec.layers):
        for qualified, role in layer_roles(layer):
            if qualified not in layer.names:
                raise KeyError(f"layer {li}: the name map has no checkpoint name for '{qualified}'")
            out[layer.names[qualified]] = role
    norm_cls = registry.norm_class(spec.final_norm.kind)
    for role in norm_cls.expected_tensors(spec.final_norm):
        # a norm has one tensor, "weight"; the final norm's checkpoint name is given whole
        out[spec.final_norm_name if role.name == "weight" else f"{spec.final_norm_name}.{role.name}"] = role
    if spec.head_name is not None:
        out[spec.head_name] = TensorRole(spec.head_name, (spec.vocab, spec.hidden), True, True)
    if spec.head_bias_name is not None:
        out[spec.head_bias_name] = TensorRole(spec.head_bias_name, (spec.vocab,), True, False, role="bias")
    return out


def check(spec: ModelSpec, shapes: Dict[str, Tuple[int, ...]], origin: str = "") -> Dict[str, TensorRole]:
    """Compare the names and shapes a checkpoint holds with what the model wants."""
    want = expected_tensors(spec)
    missing = [n for n, r in want.items() if r.required and n not in shapes]
    unexpected = [n for n in shapes if n not in want]
    wrong = [(n, tuple(shapes[n]), r.shape) for n, r in want.items()
             if n in shapes and tuple(shapes[n]) != tuple(r.shape)]
    if missing or unexpected or wrong:
        raise WeightError(sorted(missing), sorted(unexpected), wrong, origin)
    return want


def bind(spec: ModelSpec, checkpoint, origin: str = "") -> Dict[str, torch.Tensor]:
    """Checkpoint name -> CPU tensor in its stored type, after `check`."""
    shapes = {n: checkpoint.shape(n) for n in checkpoint.names()}
    want = check(spec, shapes, origin)
    return {n: checkpoint.tensor(n) for n in want if n in shapes}


class TensorDict:
    """A dict of tensors with the checkpoint's reading interface (for weights made in memory)."""

    def __init__(self, tensors: Dict[str, torch.Tensor]):
        self._t = tensors

    def names(self):
        return list(self._t)

    def shape(self, name):
        return tuple(self._t[name].shape)

    def tensor(self, name):
        return self._t[name]
