"""Weights: the safetensors container, binding by name, one error for all misfits, random mode
(no GPU)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

from beglin_b200.config import load_config
from beglin_b200.weights import (Checkpoint, SafetensorsError, WeightError, bind, check, expected_tensors,
                                 random_tensors, write_random_model, write_safetensors)
from helpers import TINY_A, TINY_B, make_model


def spec_of(cfg):
    arch, c = load_config(cfg)
    return arch.build_spec(c)


def test_random_model_folder_reads_back(model_root):
    folder = make_model(model_root, "B", seed=3, dtype=torch.bfloat16)
    assert os.path.exists(os.path.join(folder, "config.json"))
    ck = Checkpoint(folder)
    spec = spec_of(json.load(open(os.path.join(folder, "config.json"))))
    bound = bind(spec, ck)
    assert set(bound) == set(expected_tensors(spec))
    assert bound["model.embed_tokens.weight"].dtype == torch.bfloat16      # kept as stored
    assert bound["lm_head.weight"].shape == (384, 96)
    # the same folder through the independent safetensors library
    from safetensors import safe_open
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            assert torch.equal(f.get_tensor(name), bound[name]), name
    ck.close()


def test_stored_types_are_kept(tmp_path):
    t = {"a": torch.randn(3, 4), "b": torch.randn(2, 2).to(torch.bfloat16), "c": torch.randn(5).to(torch.float16),
         "i": torch.arange(6, dtype=torch.int64).reshape(2, 3)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t)
    ck = Checkpoint(p)
    assert ck.tensor("a").dtype == torch.float32 and torch.equal(ck.tensor("a"), t["a"])
    assert ck.tensor("b").dtype == torch.bfloat16 and torch.equal(ck.tensor("b"), t["b"])
    assert ck.tensor("c").dtype == torch.float16 and torch.equal(ck.tensor("c"), t["c"])
    assert ck.tensor("i").dtype == torch.int32 and ck.tensor("i").tolist() == t["i"].tolist()


def test_random_weights_are_seeded_and_independent_of_order():
    spec = spec_of(TINY_A)
    a = random_tensors(spec, 7, dtype=torch.float32)
    b = random_tensors(spec, 7, dtype=torch.float32)
    c = random_tensors(spec, 8, dtype=torch.float32)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    w = a["model.layers.0.input_layernorm.weight"]
    assert abs(float(w.mean()) - 1.0) < 0.02 and float(w.std()) < 0.05
    assert abs(float(a["model.layers.1.mlp.up_proj.weight"].std()) - 0.02) < 0.003


def test_random_weights_follow_the_role_not_the_name():
    """How a tensor is drawn is what its part says it is for.  A model whose checkpoint calls a projection
    matrix "...norm.bias" and a norm's weight "...matrix" still gets a matrix around zero and a scale around one."""
    spec = spec_of(TINY_A)
    layer = spec.layers[0]
    names = dict(layer.names)
    names["mixer.o_proj.weight"] = "odd.names.out_norm.bias"
    names["mixer_norm.weight"] = "odd.names.first.matrix"
    names["mixer.q_proj.bias"] = "odd.names.q_norm.weight"
    spec.layers[0] = layer.with_parts(names=names)
    t = random_tensors(spec, 7, std=0.02, bias_std=0.3, norm_std=0.02, dtype=torch.float32)
    assert abs(float(t["odd.names.out_norm.bias"].mean())) < 0.005 and abs(float(t["odd.names.out_norm.bias"].std()) - 0.02) < 0.004
    assert abs(float(t["odd.names.first.matrix"].mean()) - 1.0) < 0.02
    assert abs(float(t["odd.names.q_norm.weight"].std()) - 0.3) < 0.08 and abs(float(t["odd.names.q_norm.weight"].mean())) < 0.15


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    spec = spec_of(TINY_A)
    t = random_tensors(spec, 0, dtype=torch.float32)
    del t["model.layers.1.mlp.down_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.o_proj.bias"] = torch.zeros(64)
    t["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64)
    shapes = {k: tuple(v.shape) for k, v in t.items()}
    with pytest.raises(WeightError) as e:
        check(spec, shapes)
    err = e.value
    assert err.missing == ["model.layers.1.mlp.down_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.o_proj.bias"]
    assert err.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (16, 64), (32, 64))]
    msg = str(err)
    for s in ("missing (2)", "unexpected (1)", "wrong shape (1)", "expected [32, 64]"):
        assert s in msg


def test_untied_model_needs_a_head_and_tied_refuses_one():
    spec = spec_of(TINY_B)
    t = random_tensors(spec, 0)
    del t["lm_head.weight"]
    with pytest.raises(WeightError, match="lm_head.weight"):
        check(spec, {k: tuple(v.shape) for k, v in t.items()})
    spec = spec_of(TINY_A)
    t = random_tensors(spec, 0)
    t["lm_head.weight"] = torch.zeros(256, 64)
    with pytest.raises(WeightError, match="unexpected"):
        check(spec, {k: tuple(v.shape) for k, v in t.items()})


def _raw(path, header: dict, data: bytes, hlen=None):
    text = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text) if hlen is None else hlen))
        f.write(text)
        f.write(data)


def test_container_faults_are_refused(tmp_path):
    p = str(tmp_path / "bad.safetensors")
    open(p, "wb").write(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="too short"):
        Checkpoint(p)
    _raw(p, {}, b"", hlen=10**9)
    with pytest.raises(SafetensorsError, match="exceeds"):
        Checkpoint(p)
    _raw(p, {"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 16]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="outside the data section"):
        Checkpoint(p)
    _raw(p, {"t": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="does not fill"):
        Checkpoint(p)
    _raw(p, {"t": {"dtype": "Q4", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        Checkpoint(p)
    _raw(p, {"t": {"shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="lacks"):
        Checkpoint(p)
    with pytest.raises(SafetensorsError, match="could not open"):
        Checkpoint(str(tmp_path / "none.safetensors"))
    # one name twice in the header: refused, as the reference refuses it (qwen_infer.c:345-350)
    entry = '{"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}'
    text = ('{"t": ' + entry + ', "u": ' + entry + ', "t": ' + entry + '}').encode()
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", len(text)) + text + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="duplicate tensor name in the header: t"):
        Checkpoint(p)


def test_sharded_folder(tmp_path):
    spec = spec_of(TINY_A)
    t = random_tensors(spec, 1, dtype=torch.float32)
    names = sorted(t)
    half = len(names) // 2
    write_safetensors(str(tmp_path / "s1.safetensors"), {n: t[n] for n in names[:half]})
    write_safetensors(str(tmp_path / "s2.safetensors"), {n: t[n] for n in names[half:]})
    wm = {n: ("s1.safetensors" if i < half else "s2.safetensors") for i, n in enumerate(names)}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    ck = Checkpoint(str(tmp_path))
    bound = bind(spec, ck)
    assert all(torch.equal(bound[n], t[n]) for n in names)
    wm[names[0]] = "../evil.safetensors"
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    with pytest.raises(SafetensorsError, match="plain file name"):
        Checkpoint(str(tmp_path))
    wm[names[0]] = "s2.safetensors"
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    with pytest.raises(SafetensorsError, match="shard lacks"):
        Checkpoint(str(tmp_path))


def test_counter_generator_is_a_function_of_seed_name_and_element():
    """The counter-based generator: any part of a tensor can be made alone, tensors do not depend on one another,
    and the values are what the formula says (checked here with Python integers for a few elements)."""
    from beglin_b200.weights import counter_random as cr
    key = cr.tensor_key(5, "model.layers.1.mlp.down_proj.weight")
    assert key != cr.tensor_key(6, "model.layers.1.mlp.down_proj.weight") != cr.tensor_key(5, "model.layers.1.mlp.up_proj.weight")
    x = cr.standard(key, 4096)
    assert np.array_equal(cr.standard(key, 100, start=1234), x[1234:1334])
    mask = (1 << 64) - 1

    def mix(z):
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
        return z ^ (z >> 31)
    for i in (0, 1, 77, 4095):
        total = 0
        for j in range(3):
            h = mix((key + (3 * i + j) * cr.GOLDEN) & mask)
            total += (h & 0xFFFF) + ((h >> 16) & 0xFFFF) + ((h >> 32) & 0xFFFF) + (h >> 48)
        assert x[i] == np.float32(total - 6 * 65535) * np.float32(1.0 / 65536.0)
    big = cr.standard(key, 1 << 20)
    assert abs(float(big.mean())) < 5e-3 and abs(float(big.std()) - 1.0) < 5e-3 and float(np.abs(big).max()) <= 6.0
    spec = spec_of(TINY_A)
    a = random_tensors(spec, 7, std=0.02, bias_std=0.3, norm_std=0.02, dtype=torch.float32, generator="counter")
    b = random_tensors(spec, 7, std=0.02, bias_std=0.3, norm_std=0.02, dtype=torch.float32, generator="counter")
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert abs(float(a["model.norm.weight"].mean()) - 1.0) < 0.02
    assert 0.2 < float(a["model.layers.0.self_attn.q_proj.bias"].std()) < 0.4
    assert 0.015 < float(a["model.layers.0.mlp.up_proj.weight"].std()) < 0.025
    with pytest.raises(ValueError, match="generator"):
        random_tensors(spec, 7, generator="dice")
