"""This framework's readers and the plain implementation against outputs of the reference's own C
code (no GPU): the fields hf_config.c reads from config.json, the per-tensor checksums of
safetensors_load.c + safetensors_quants.c, and the frequency ratios of rope_llama3_scale.h.  The
golden files were made by tests/golden/make_golden.py; where the variable BEGLIN_REFERENCE names the
reference tree and gcc is present, the programs are also compiled and run afresh."""
import json
import os
import shutil
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
        assert abs(r - m) < 2e-6 and abs(r - o) < 2e-6       # the header computes in float


@pytest.mark.skipif(not (os.path.isdir(REF) and shutil.which("gcc")), reason="reference tree or gcc not present")
def test_fresh_run_of_the_reference_programs_agrees_with_the_golden_files(folders, tmp_path):
    tools = mg.build_tools(REF, str(tmp_path))
    for name, _, _ in mg.CASES:
        outs = mg.run_tools(tools, folders[name])
        for kind, text in outs.items():
            assert text == golden(kind, name), (kind, name)
