"""Portions of one request whose shape comes again are replayed as a CUDA graph: the replayed steps give
the rows of the uncaptured step (bitwise in float32), for other requests and other places in the context
than the ones the graph was captured with, over pages that were used before, and with a window."""
import pytest
import torch

import replay_lib as rl
from helpers import TINY, TOL_BF16, TOL_F32, make_model, plain_logits, rel_err, seeded_ids

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("B", "bfloat16"), ("C", "float32"), ("D", "bfloat16")])
def test_replayed_portions_equal_uncaptured_steps(model_root, name, dtype):
    from beglin_b200 import Engine
    cfg, _, page = TINY[name]
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = make_model(model_root, name, seed=11, dtype=stored)
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    rows, n = 24, 5
    ids = {r: seeded_ids(rows * n, cfg["vocab_size"], 70 + i) for i, r in enumerate("abc")}
    want = [0, 7, rows - 1]

    def portions(eng, rid):
        out = []
        for k in range(n):
            out.append(eng.step([(rid, ids[rid][k * rows:(k + 1) * rows], want)], end=[rid] if k == n - 1 else []))
        return torch.cat(out)

    plain_rows = [k * rows + w for k in range(n) for w in want]
    # without graphs: the rows to compare with
    eager = Engine.from_folder(folder, dtype=dtype, max_tokens=192, page_size=page, max_requests=2, use_graphs=False)
    rl.poison(eager)
    ref = {r: portions(eager, r) for r in "abc"}
    assert eager.portions.replays == 0
    for r in "abc":
        assert rel_err(ref[r], plain_logits(folder, ids[r])[plain_rows]) < tol
    del eager
    # with graphs from 8 rows on: the first portion runs kernel by kernel, the second captures, the rest replay;
    # requests b and c are replayed from their first portion on, over the pages that a gave back
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=192, page_size=page, max_requests=2, portion_graph_rows=8)
    rl.poison(eng)
    for r in "abc":
        got = portions(eng, r)
        assert torch.isfinite(got).all()
        if dtype == "float32":
            assert torch.equal(got, ref[r]), r
        else:
            assert rel_err(got, plain_logits(folder, ids[r])[plain_rows]) < tol, r
    assert eng.portions.replays == 3 * n - 1
    assert len(eng.portions.graphs) == 1
    # a step of two requests, a shape with many wanted places and a short portion run without a graph
    before = eng.portions.replays
    eng.step([("d", ids["a"][:rows], want), ("e", ids["b"][:rows], want)], end=["d", "e"])
    eng.step([("d", ids["a"][:rows], list(range(rows)))], end=["d"])
    eng.step([("d", ids["a"][:4], [3])], end=["d"])
    eng.step([("d", ids["a"][:4], [3])], end=["d"])
    assert eng.portions.replays == before
    eng.cache.check()


def test_least_recently_used_graphs_are_dropped(model_root):
    from beglin_b200 import Engine
    cfg, _, page = TINY["A"]
    folder = make_model(model_root, "A", seed=11, dtype=torch.float32)
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=128, page_size=page, max_requests=2, portion_graph_rows=8)
    eng.portions.keep = 2
    ids = seeded_ids(40, cfg["vocab_size"], 5)
    want = plain_logits(folder, ids)
    for rows in (10, 12, 14, 10):
        for _ in range(3):
            got = eng.step([("a", ids[:rows], [rows - 1])], end=["a"])
            assert rel_err(got, want[[rows - 1]]) < TOL_F32
    assert len(eng.portions.graphs) == 2 and [k[0] for k in eng.portions.graphs] == [14, 10]
