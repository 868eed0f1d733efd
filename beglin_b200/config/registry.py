"""The one registry from an architecture's name to its configuration class and model spec.

The name is `architectures[0]` of config.json; a folder without that key is resolved through
`model_type` (the reference's C engine keys on `model_type` alone, qwen_infer.c:18989 and
:19360-19372, and its Python registry falls back to `architectures[0]`,
tools/model_capability.py:793-815).  An unknown name is an error that lists the names known,
in the manner of qwen_infer.c:19369.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional

from .reader import ConfigError, ConfigFields


@dataclass(frozen=True)
class Architecture:
    name: str
    model_type: str
    config_class: type                 # has from_fields(ConfigFields, tensor_names=None)
    build_spec: Callable               # config -> parts.spec.ModelSpec


ARCHITECTURES: Dict[str, Architecture] = {}
_MODEL_TYPES: Dict[str, str] = {}


def register_architecture(arch: Architecture) -> Architecture:
    ARCHITECTURES[arch.name] = arch
    _MODEL_TYPES[arch.model_type] = arch.name
    return arch


def resolve_architecture(fields: ConfigFields) -> Architecture:
    names = fields.string_list("architectures")
    model_type = fields.string("model_type")
    name: Optional[str] = None
    if names:
        name = names[0]
    elif model_type is not None:
        name = _MODEL_TYPES.get(model_type, model_type)
    if name is None:
        raise ConfigError(f"{fields.origin} missing 'architectures' and 'model_type'")
    arch = ARCHITECTURES.get(name)
    if arch is None:
        known = ", ".join(sorted(ARCHITECTURES))
        raise ConfigError(f"{fields.origin}: architecture '{name}' not validated by this engine; supported: {known}")
    if model_type is not None and model_type != arch.model_type:
        raise ConfigError(f"{fields.origin}: model_type '{model_type}' does not belong to architecture "
                          f"'{name}' (expected '{arch.model_type}')")
    return arch
