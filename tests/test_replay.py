"""Replay of the same requests in four ways of cutting and batching, in float32 and bfloat16,
against the plain implementation: whole; most in one step and the last 32 tokens one by one; in
portions of changing size down to two tokens; and mixed, up to four live requests on a pool so
small that pages are used again.  In float32 every kernel sums each output in an order that does
not depend on the batch, so the four ways must agree bit for bit."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import replay_lib as rl
from helpers import TINY, TOL_BF16, TOL_F32, make_model, plain_logits, rel_err, seeded_ids

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [70, 45, 100, 33, 120, 64], "B": [130, 33, 250, 97, 64, 180], "C": [300, 41, 150, 90, 270, 65],
           "D": [300, 41, 150, 90, 270, 65]}


def requests_for(name):
    cfg = TINY[name][0]
    return {f"r{i}": seeded_ids(n, cfg["vocab_size"], 100 + i) for i, n in enumerate(LENGTHS[name])}


def engine_for(folder, dtype, max_tokens, page_size, kv_split=64):
    from beglin_b200 import Engine
    e = Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, page_size=page_size, max_requests=4,
                           kv_split=kv_split)
    rl.poison(e)
    return e


def check_against_plain(got, folder, reqs, tol):
    worst = 0.0
    for rid, ids in reqs.items():
        want = plain_logits(folder, ids)
        rows = torch.stack([got[(rid, p)] for p in range(len(ids))])
        assert torch.isfinite(rows).all(), rid
        err = rel_err(rows, want)
        if err > tol:
            per_pos = (rows.double() - want).abs().max(dim=1).values / want.abs().max()
            first = int((per_pos > tol).nonzero()[0])
            raise AssertionError(f"{rid}: relative error {err:.3g} > {tol:g}; first wrong position {first} of {len(ids)}")
        worst = max(worst, err)
    return worst


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_four_ways_of_cutting(model_root, name, dtype):
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = make_model(model_root, name, seed=11, dtype=stored)
    page = TINY[name][2]
    reqs = requests_for(name)
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    mixed_steps, peak = rl.mixed(reqs, seed=5)
    results = {}
    for way, steps, max_tokens in (("whole", rl.whole(reqs), 320), ("tail", rl.last_one_by_one(reqs), 320),
                                   ("portions", rl.portions(reqs), 320), ("mixed", mixed_steps, peak)):
        eng = engine_for(folder, dtype, max_tokens, page, kv_split=64 if name in "AB" else 256)
        got = rl.run_in_process(eng, steps)
        eng.cache.check()
        assert eng.cache.free_pages() == eng.cache.num_pages and not eng.cache.live()
        worst = check_against_plain(got, folder, reqs, tol)
        print(f"{name} {dtype} {way}: worst relative error {worst:.3g} (limit {tol:g})")
        results[way] = got
        del eng
    if dtype == "float32":
        for way in ("tail", "portions", "mixed"):
            for key, row in results["whole"].items():
                assert torch.equal(row, results[way][key]), (way, key)


def test_pages_are_really_used_again(model_root):
    folder = make_model(model_root, "A", seed=11, dtype=torch.float32)
    reqs = requests_for("A")
    steps, peak = rl.mixed(reqs, seed=5)
    assert peak < sum(-(-len(v) // 64) * 64 for v in reqs.values())       # the pool cannot hold all at once
    eng = engine_for(folder, "float32", peak, 8)
    seen, reused = set(), False
    for s in steps:
        eng.step(s["entries"], end=[])
        for e in s["entries"]:
            pages = {p for p in eng.cache.kv_groups[0].tables[e["id"]] if p >= 0}
            reused = reused or any(p in seen for p in pages)
        for rid in s["end"]:
            seen |= {p for p in eng.cache.kv_groups[0].tables[rid] if p >= 0}
            eng.release(rid)
    assert reused


def test_first_tokens_of_a_sequence(model_root):
    """Positions 0, 1, 2 alone: a single token, then one more, then a portion of two."""
    for name, dtype, tol in (("A", "float32", TOL_F32), ("B", "bfloat16", TOL_BF16)):
        stored = torch.float32 if dtype == "float32" else torch.bfloat16
        folder = make_model(model_root, name, seed=11, dtype=stored)
        ids = seeded_ids(5, TINY[name][0]["vocab_size"], 9)
        eng = engine_for(folder, dtype, 64, TINY[name][2])
        steps = [{"entries": [{"id": "x", "tokens": ids[:1], "want": [0]}]},
                 {"entries": [{"id": "x", "tokens": ids[1:2], "want": [0]}]},
                 {"entries": [{"id": "x", "tokens": ids[2:4], "want": [0, 1]}]},
                 {"entries": [{"id": "x", "tokens": ids[4:5], "want": [0]}], "end": ["x"]}]
        got = rl.run_in_process(eng, steps)
        check_against_plain(got, folder, {"x": ids}, tol)


def test_long_decoding(model_root):
    """A short prompt, then 280 tokens one by one across page and split boundaries, beside a second
    request that decodes too."""
    folder = make_model(model_root, "C", seed=11, dtype=torch.float32)
    vocab = TINY["C"][0]["vocab_size"]
    a, b = seeded_ids(290, vocab, 21), seeded_ids(200, vocab, 22)
    eng = engine_for(folder, "float32", 576, 16, kv_split=64)
    steps = [{"entries": [{"id": "a", "tokens": a[:10], "want": [9]}, {"id": "b", "tokens": b[:3], "want": [2]}]}]
    for i in range(10, 290):
        ents = [{"id": "a", "tokens": [a[i]], "want": [0]}]
        j = i - 7
        if j < 200:
            ents.append({"id": "b", "tokens": [b[j]], "want": [0]})
        steps.append({"entries": ents, "end": []})
    got = rl.run_in_process(eng, steps)
    wa, wb = plain_logits(folder, a), plain_logits(folder, b)
    for (rid, p), row in got.items():
        want = (wa if rid == "a" else wb)[p]
        assert rel_err(row, want) < TOL_F32, (rid, p)


def test_bad_input_is_refused(model_root):
    folder = make_model(model_root, "A", seed=11, dtype=torch.float32)
    eng = engine_for(folder, "float32", 64, 8)
    with pytest.raises(ValueError, match="vocabulary"):
        eng.step([("x", [1, 256], [0])])
    with pytest.raises(ValueError, match="wanted place"):
        eng.step([("x", [1, 2], [2])])
    with pytest.raises(ValueError, match="twice"):
        eng.step([("x", [1], []), ("x", [2], [])])
    from beglin_b200.cache import OutOfPages
    with pytest.raises(OutOfPages):
        eng.step([("x", list(range(60)), []), ("y", list(range(10)), [])])
    assert not eng.cache.live() and eng.cache.free_pages() == eng.cache.num_pages
    assert eng.step([("x", [1, 2, 3], [])]) is None           # nothing wanted: no logits, the head is skipped


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(model_root, tmp_path, dtype):
    """bin/trace_run as a user runs it: JSON lines in, <step>.f32 files out, `done <step>` after each."""
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = make_model(model_root, "B", seed=11, dtype=stored)
    reqs = {k: v for k, v in list(requests_for("B").items())[:4]}
    steps, peak = rl.mixed(reqs, seed=8)
    steps = rl.number(steps)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    cmd = [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
           "--out", str(out), "--max-tokens", str(peak)]
    text = "".join(json.dumps(s) + "\n" for s in steps)
    r = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    vocab = TINY["B"][0]["vocab_size"]
    got, held = {}, {}
    for s in steps:
        n_want = sum(len(e["want"]) for e in s["entries"])
        path = out / f"{s['step']}.f32"
        if n_want == 0:
            assert not path.exists()
            continue
        arr = np.fromfile(path, dtype="<f4").reshape(n_want, vocab)
        row = 0
        for e in s["entries"]:
            start = held.get(e["id"], 0)
            for w in e["want"]:
                got[(e["id"], start + w)] = torch.from_numpy(arr[row].copy())
                row += 1
            held[e["id"]] = start + len(e["tokens"])
    check_against_plain(got, folder, reqs, TOL_F32 if dtype == "float32" else TOL_BF16)
