"""This framework's readers and the plain implementation against outputs of the reference's own C
code (no GPU): the fields hf_config.c reads from config.json, the per-tensor checksums of
safetensors_load.c + safetensors_quants.c, the frequency ratios of rope_llama3_scale.h, and tiny random
models run token by token by the functions of qwen_infer.c's own arithmetic (norm, softmax, SwiGLU,
rotation, the plain attention loop, argmax; see tests/golden/make_golden.py).  The
golden files were made by tests/golden/make_golden.py; where the variable BEGLIN_REFERENCE names the
reference tree and gcc is present, the programs are also compiled and run afresh."""
import json
import os
import shutil
import struct
import sys

import pytest
import torch

from helpers import plain

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_golden as mg  # noqa: E402

REF = os.environ.get("BEGLIN_REFERENCE", "")           # the reference tree, when the caller has one


def golden(kind, name):
    with open(os.path.join(HERE, "golden", f"{kind}_{name}.txt")) as f:
        return f.read()


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("golden"))
    return {name: mg.case_folder(root, name, seed, dtype) for name, seed, dtype in mg.CASES}


def config_lines(folder):
    """What hf_config_verify.c prints, from this framework's typed configuration."""
    from beglin_b200.config import load_config
    _, c = load_config(folder)
    raw = json.load(open(os.path.join(folder, "config.json")))
    out = [f"hidden_size={c.hidden_size}", f"num_hidden_layers={c.num_hidden_layers}",
           f"intermediate_size={c.intermediate_size}", f"num_attention_heads={c.num_attention_heads}",
           f"num_key_value_heads={c.num_key_value_heads}", f"rms_norm_eps={c.rms_norm_eps:.9g}",
           f"rope_theta={c.rope_theta:.9g}", f"vocab_size={c.vocab_size}",
           f"tie_word_embeddings={'true' if c.tie_word_embeddings else 'false'}", f"model_type={c.model_type}"]
    if c.max_position_embeddings is not None:
        out.append(f"max_position_embeddings={c.max_position_embeddings}")
    if c.rope_scaling is None:
        out.append("rope_scaling=" + ("NULL" if "rope_scaling" in raw else "ABSENT"))
    else:
        r = c.rope_scaling
        out += ["rope_scaling=OBJECT", "rope_scaling.rope_type=llama3", f"rope_scaling.factor={r.factor:.9g}",
                f"rope_scaling.low_freq_factor={r.low_freq_factor:.9g}",
                f"rope_scaling.high_freq_factor={r.high_freq_factor:.9g}",
                f"rope_scaling.original_max_position_embeddings={r.original_max_position_embeddings}"]
    return out


def checksums(folder):
    """safetensors_verify.c's weighted checksum, from this framework's container reader."""
    from beglin_b200.weights import Checkpoint
    ck = Checkpoint(folder)
    out = {}
    for name in ck.names():
        t = ck.tensor(name).double().reshape(-1)
        wgt = (torch.arange(t.numel(), dtype=torch.float64) % 97) + 1.0
        out[name] = (float((t * wgt).sum()), t.numel(), ck.dtype(name))
    ck.close()
    return out


def parse_checksums(text):
    out = {}
    for line in text.strip().splitlines():
        name, cs, n, dt = line.split()
        out[name] = (float(cs.split("=")[1]), int(n.split("=")[1]), dt.split("=")[1])
    return out


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_config_fields_match_the_reference_reader(folders, name):
    assert config_lines(folders[name]) == golden("config", name).strip().splitlines()


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_tensor_checksums_match_the_reference_reader(folders, name):
    mine, ref = checksums(folders[name]), parse_checksums(golden("checksums", name))
    assert set(mine) == set(ref)
    for k, (cs, n, dt) in ref.items():
        assert mine[k][1] == n and mine[k][2] == dt, k
        assert abs(mine[k][0] - cs) <= 1e-6 * max(1.0, abs(cs)), (k, mine[k][0], cs)


def test_frequency_ratios_match_the_reference_header(folders):
    from beglin_b200.config import load_config
    from beglin_b200.models.qwen2 import llama3_frequency_scale
    _, c = load_config(folders["C"])
    ref = [float(l.split()[1]) for l in golden("rope_scale", "C").strip().splitlines()]
    mine = llama3_frequency_scale(c.rope_theta, c.head_dim, c.rope_scaling)
    oracle = plain.frequency_scale(json.load(open(os.path.join(folders["C"], "config.json"))), c.head_dim)
    assert len(ref) == len(mine) == c.head_dim // 2
    for r, m, o in zip(ref, mine, oracle.tolist()):
        # the header computes in float, and so do both restatements: the same 32-bit numbers (nine digits name one)
        assert struct.pack("<f", r) == struct.pack("<f", m) == struct.pack("<f", o), (r, m, o)


def parse_model_golden(name):
    rope, logits, greedy, other = {}, {}, [], {}
    for line in golden("model", name).strip().splitlines():
        kind, *rest = line.split()
        if kind == "rope":
            v = torch.tensor([float(x) for x in rest[1:]], dtype=torch.float64)
            rope[int(rest[0])] = (v[0::2], v[1::2])
        elif kind == "logits":
            logits[int(rest[0])] = torch.tensor([float(x) for x in rest[1:]], dtype=torch.float64)
        elif kind == "greedy":
            greedy.append(int(rest[1]))
        else:
            other[kind] = float(rest[0])
    return rope, logits, greedy, other


@pytest.mark.parametrize("case", mg.MODEL_CASES, ids=[c[0] for c in mg.MODEL_CASES])
def test_plain_model_matches_the_reference_functions(tmp_path, case):
    """The plain implementation (float64) against the reference's own compiled arithmetic (float): logits of three
    positions of a seeded sequence, the greedy continuation, and the rotation's cosines and sines up to position
    32,767.  The tolerances are those of float arithmetic: 2e-5 of the largest logit; 1e-6 for a cosine."""
    name, seed, dtype, ids_seed, n, n_new = case
    folder = mg.model_case_folder(str(tmp_path), name, seed, dtype)
    ids = mg.model_case_ids(name, ids_seed, n)
    rope, logits, greedy, other = parse_model_golden(name)
    cfg, w = plain.read_folder(folder, torch.float64)
    assert sorted(logits) == sorted({0, n // 2, n - 1}) and len(greedy) == n_new and other["rope_head_vs_apply"] == 0.0
    mine = plain.forward(cfg, w, ids + greedy[:-1])
    for pos, row in logits.items():
        assert float((mine[pos] - row).abs().max()) < 2e-5 * float(row.abs().max()), (name, pos)
    # the greedy tokens: where the reference's top two logits are a float's rounding apart either may win
    for k, tok in enumerate(greedy):
        row = mine[n - 1 + k]
        assert plain.greedy_token(row) == tok or float(row.max() - row[tok]) < 2e-5 * float(row.abs().max()), (name, k)
    sz = plain.sizes(cfg)
    for pos, (c, s_) in rope.items():
        ang = plain.rope_angles([pos], sz["hd"], cfg["rope_theta"], torch.float64, plain.frequency_scale(cfg, sz["hd"]))[0]
        assert float((torch.cos(ang) - c).abs().max()) < 1e-6 and float((torch.sin(ang) - s_).abs().max()) < 1e-6, (name, pos)


def test_engine_frequencies_are_the_reference_numbers():
    """The rotary part's 32-bit frequencies give the reference's cosines at position 32,767 (where one unit in a
    frequency's last place would move the angle by 0.002)."""
    from beglin_b200.parts.context import BuildContext
    from beglin_b200.parts.rope import RotaryPosition
    from beglin_b200.config import load_config
    for name in ("A", "B", "Cfull"):
        arch, c = load_config(mg.model_case_config(name))
        position = arch.build_spec(c).layers[0].mixer.position
        part = RotaryPosition(position, BuildContext(device="cpu", compute_dtype=torch.float32))
        rope = parse_model_golden(name)[0]
        for pos, (cos, sin) in rope.items():
            ang = (torch.tensor(float(pos), dtype=torch.float32) * part.inv_freq).double()      # the kernel's float product
            assert float((torch.cos(ang) - cos).abs().max()) < 1e-6 and float((torch.sin(ang) - sin).abs().max()) < 1e-6, (name, pos)


@pytest.mark.skipif(not (os.path.isdir(REF) and shutil.which("gcc")), reason="reference tree or gcc not present")
def test_fresh_run_of_the_reference_programs_agrees_with_the_golden_files(folders, tmp_path):
    tools = mg.build_tools(REF, str(tmp_path))
    for name, _, _ in mg.CASES:
        outs = mg.run_tools(tools, folders[name])
        for kind, text in outs.items():
            assert text == golden(kind, name), (kind, name)
    for name, seed, dtype, ids_seed, n, n_new in mg.MODEL_CASES:
        folder = mg.model_case_folder(str(tmp_path), name, seed, dtype)
        text = mg.run_model_driver(tools["model"], folder, str(tmp_path), mg.model_case_ids(name, ids_seed, n), n_new)
        assert text == golden("model", name), name
