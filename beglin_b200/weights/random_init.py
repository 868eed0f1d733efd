"""Random weights for a configuration: in memory, or as a model folder (config.json and
model.safetensors) that every loader of the framework reads like a downloaded one.

Matrices and biases are N(0, std) and N(0, bias_std); norm weights are 1 + N(0, norm_std); which
of these a tensor is says the `role` of the part's `TensorRole`, never its name.  Each
tensor has a generator of its own, seeded from (seed, tensor name), so the values do not depend on
the order or on which other tensors exist.  The reference has no such mode in its engine; its tests
write a seeded three-tensor fixture (tests/regression/mk_tiny_st.py:21-45).

Two generators.  "torch": the host library's normal generator (the default of the folder writer).
"counter": a counter-based one (counter_random.py), element i a function of (seed, name, i) alone, which
numpy on the host and a fill kernel on the device compute to the same bits: weights made on the device
(`Engine.random`, sizes too large to write to disk first) are then the weights of the folder that the same
seed writes with generator="counter", and an oracle can be run on the host against an engine that never saw a file.
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Dict, Optional

import torch

from ..parts.spec import ModelSpec
from .loader import expected_tensors
from .safetensors_io import write_safetensors


def _counter_tensor(name: str, role, seed: int, mean: float, scale: float, dtype: torch.dtype, device: str) -> torch.Tensor:
    from . import counter_random
    key = counter_random.tensor_key(seed, name)
    if device != "cpu":
        from ..csrc import ops
        t = torch.empty(role.shape, dtype=dtype, device=device)
        ops.fill_normal(t, key, mean, scale)
        return t
    n = 1
    for d in role.shape:
        n *= int(d)
    t = torch.empty(n, dtype=dtype)
    step = 1 << 22                          # in pieces, so that a large table's 64-bit intermediates stay small
    for i0 in range(0, n, step):
        m = min(step, n - i0)
        t[i0:i0 + m] = torch.from_numpy(counter_random.normal(key, m, mean, scale, start=i0)).to(dtype)
    return t.reshape(role.shape)


def random_tensors(spec: ModelSpec, seed: int, std: float = 0.02, bias_std: Optional[float] = None,
                   norm_std: float = 0.02, dtype: torch.dtype = torch.bfloat16,
                   device: str = "cpu", generator: str = "torch") -> Dict[str, torch.Tensor]:
    if generator not in ("torch", "counter"):
        raise ValueError(f"generator must be 'torch' or 'counter', got {generator!r}")
    bias_std = std if bias_std is None else bias_std
    out: Dict[str, torch.Tensor] = {}
    for name, role in expected_tensors(spec).items():
        if generator == "counter":
            kind = role.init_role()
            mean, scale = (1.0, norm_std) if kind == "scale" else (0.0, bias_std if kind == "bias" else std)
            out[name] = _counter_tensor(name, role, seed, mean, scale, dtype, device)
            continue
        gen = torch.Generator(device=device)
        gen.manual_seed((int(seed) * 1000003 + zlib.crc32(name.encode())) % (2**63))
        kind = role.init_role()            # what the part says the tensor is for; the checkpoint's name plays no part
        if role.matrix and device != "cpu" and len(role.shape) == 2 and role.shape[0] * role.shape[1] > (1 << 26):
            # large tables are filled in row blocks so the float32 draw never doubles their footprint
            t = torch.empty(role.shape, dtype=dtype, device=device)
            step = max(1, (1 << 26) // role.shape[1])
            for r0 in range(0, role.shape[0], step):
                r1 = min(role.shape[0], r0 + step)
                t[r0:r1] = (torch.randn((r1 - r0, role.shape[1]), generator=gen, device=device) * std).to(dtype)
            out[name] = t
            continue
        x = torch.randn(role.shape, generator=gen, dtype=torch.float32, device=device)
        if kind == "scale":
            x = 1.0 + norm_std * x
        elif kind == "bias":
            x = bias_std * x
        else:
            x = std * x
        out[name] = x.to(dtype)
    return out


def write_random_model(folder: str, config_json: dict, seed: int, std: float = 0.02,
                       bias_std: Optional[float] = None, norm_std: float = 0.02,
                       dtype: torch.dtype = torch.bfloat16, generator: str = "torch") -> str:
    """Write `folder`/config.json and `folder`/model.safetensors for the configuration given as
    config.json keys.  Returns the folder."""
    from ..config import load_config
    arch, cfg = load_config(dict(config_json))
    spec = arch.build_spec(cfg)
    tensors = random_tensors(spec, seed, std, bias_std, norm_std, dtype, generator=generator)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config_json, f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed), "generator": generator})
    return folder
