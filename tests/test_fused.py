"""Steps of few tokens run the fused products (norm inside the product, residual add and SwiGLU behind it).
They must agree with the plain way (every norm, add and SwiGLU a kernel of its own) and with the oracle."""
import pytest
import torch

import replay_lib as rl
from helpers import TINY, TOL_BF16, make_model, plain_logits, rel_err, seeded_ids

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_fused_and_plain_steps_agree(model_root, name):
    from beglin_b200 import Engine
    cfg, _, page = TINY[name]
    folder = make_model(model_root, name, seed=11, dtype=torch.bfloat16)
    ids = seeded_ids(40, cfg["vocab_size"], 5)
    want = plain_logits(folder, ids)
    outs = {}
    for fuse in (True, False, "all"):
        eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=256, page_size=page, max_requests=2, fuse=fuse)
        rl.poison(eng)
        layer = eng.model.blocks[0]
        assert layer.mixer.qkv.fuses(4) == bool(fuse) and layer.feed_forward.down.fuses(4) == bool(fuse)
        assert not layer.mixer.qkv.fuses(17)                       # only few-token steps
        # rotation and cache append inside the q/k/v product: for heads that fit its tiles; a product of as few CTAs
        # as these models' only when everything is fused that can be
        hd = layer.mixer.hd
        assert (layer.mixer.rope_in_product and layer.mixer.qkv.rope_fuses(4, hd)) == (fuse == "all" and hd in (32, 64, 128))
        rows = [eng.step([("r", ids[:20], list(range(20)))])]      # a portion (plain way in both engines)
        for t in range(20, 40, 4):                                 # then four tokens at a time (fused when allowed)
            rows.append(eng.step([("r", ids[t:t + 4], [0, 1, 2, 3])]))
        outs[fuse] = torch.cat(rows).cpu()
        assert rel_err(outs[fuse], want) < TOL_BF16, (name, fuse)
    assert rel_err(outs[True], outs[False]) < TOL_BF16 / 2
    assert rel_err(outs["all"], outs[False]) < TOL_BF16 / 2
    assert torch.equal(outs[True][:20], outs[False][:20])          # the portion ran the same kernels
    assert torch.equal(outs["all"][:20], outs[False][:20])


def test_fused_swiglu_needs_blocks_of_64(model_root):
    from beglin_b200 import Engine
    for name, block in (("A", 64), ("B", 0)):                      # intermediate sizes 128 and 200
        folder = make_model(model_root, name, seed=3, dtype=torch.bfloat16)
        eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=128, page_size=TINY[name][2], max_requests=1)
        assert eng.model.blocks[0].feed_forward.block == block


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_pages_of_64_positions(model_root, dtype):
    """The engine's default page size (a page is a tile of the attention kernels and comes in one TMA box):
    a prompt in portions, then token by token across a page's edge, with a second request in between."""
    from beglin_b200 import Engine
    from helpers import TOL_F32
    cfg, _, _ = TINY["D"]
    stored = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    folder = make_model(model_root, "D", seed=13, dtype=stored)
    ids = {"a": seeded_ids(150, cfg["vocab_size"], 7), "b": seeded_ids(70, cfg["vocab_size"], 8)}
    want = {r: plain_logits(folder, ids[r]) for r in ids}
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=256, max_requests=2)       # 4 pages of 64
    assert eng.cache.page_size == 64
    rl.poison(eng)
    got = {"a": [], "b": []}
    got["a"].append(eng.step([("a", ids["a"][:60], list(range(60)))]))
    got["b"].append(eng.step([("b", ids["b"][:3], [0, 1, 2])]))
    for t in range(60, 70):                                    # across the edge at 64, beside the other request
        out = eng.step([("a", ids["a"][t:t + 1], [0]), ("b", ids["b"][t - 57:t - 56], [0])])
        got["a"].append(out[:1]); got["b"].append(out[1:])
    got["a"].append(eng.step([("a", ids["a"][70:150], list(range(80)))], end=["a"]))   # a third page; then its pages go back
    got["b"].append(eng.step([("b", ids["b"][13:70], list(range(57)))], end=["b"]))
    tol = TOL_BF16 if dtype == "bfloat16" else TOL_F32
    for r in ids:
        assert rel_err(torch.cat(got[r]).cpu(), want[r]) < tol, r
    eng.cache.check()


def test_steps_of_many_rows_run_swiglu_inside_the_pair_product(model_root):
    """From 192 rows on, gate/up and SwiGLU are one kernel of CTA pairs.  A whole prompt of 300 tokens, then a step of
    a 200-token portion of a second request beside a decoded token of the first, then the rest (under 192 rows: the
    library's product and the SwiGLU kernel), against the plain implementation and against an engine without fusions."""
    from beglin_b200 import Engine
    cfg = dict(TINY["D"][0], intermediate_size=320, num_hidden_layers=3, use_sliding_window=False)
    folder = make_model(model_root, "pairs", seed=21, dtype=torch.bfloat16, config=cfg, std=0.05, bias_std=0.05)
    ids = {"a": seeded_ids(301, cfg["vocab_size"], 3), "b": seeded_ids(300, cfg["vocab_size"], 4)}
    want = {r: plain_logits(folder, ids[r]) for r in ids}
    outs = {}
    for fuse in (True, False):
        eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=1024, max_requests=2, fuse=fuse)
        rl.poison(eng)
        ff = eng.model.blocks[0].feed_forward
        assert ff.block == 64 and ff.gate_up._tc.pairs(192) == fuse and not ff.gate_up._tc.pairs(191)
        got = {"a": [], "b": []}
        got["a"].append(eng.step([("a", ids["a"][:300], list(range(300)))]))
        out = eng.step([("b", ids["b"][:200], list(range(200))), ("a", ids["a"][300:], [0])])
        got["b"].append(out[:200]); got["a"].append(out[200:])
        got["b"].append(eng.step([("b", ids["b"][200:], list(range(100)))]))
        outs[fuse] = {r: torch.cat(got[r]).cpu() for r in ids}
        for r in ids:
            assert rel_err(outs[fuse][r], want[r]) < TOL_BF16, (r, fuse)
    for r in ids:
        assert rel_err(outs[True][r], outs[False][r]) < TOL_BF16 / 2


def test_an_engine_of_own_products_only(model_root):
    """gemm="tcgen05": every product of the model on this package's kernels; steps of 192 rows and more then run
    the products of CTA pairs in all three modes (plain with bias for q/k/v, into the residual stream for the
    output and down products, SwiGLU for gate/up).  Against the plain implementation and the default engine."""
    from beglin_b200 import Engine
    cfg = dict(TINY["D"][0], intermediate_size=320, num_hidden_layers=3, use_sliding_window=False)
    folder = make_model(model_root, "pairs", seed=21, dtype=torch.bfloat16, config=cfg, std=0.05, bias_std=0.05)
    ids = seeded_ids(330, cfg["vocab_size"], 9)
    want = plain_logits(folder, ids)
    outs = {}
    for gemm in ("tcgen05", "auto"):
        eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=512, max_requests=1, gemm=gemm)
        rl.poison(eng)
        got = [eng.step([("a", ids[:250], list(range(250)))]), eng.step([("a", ids[250:270], list(range(20)))]),
               eng.step([("a", ids[270:], list(range(60)))])]
        outs[gemm] = torch.cat(got).cpu()
        assert rel_err(outs[gemm], want) < TOL_BF16, gemm
    assert rel_err(outs["tcgen05"], outs["auto"]) < TOL_BF16 / 2


@pytest.mark.parametrize("name", ["B", "D"])
def test_everything_fused_in_a_mixed_replay(model_root, name):
    """Up to four live requests, portions of some beside decoded tokens of others, a pool so small that pages are
    used again, with every fusion on that the sizes allow: the rope epilogue of the q/k/v product among them, which
    products as small as these models' do not get by default.  Heads of 32 (B) and 64 (D)."""
    from beglin_b200 import Engine
    cfg, _, page = TINY[name]
    folder = make_model(model_root, name, seed=17, dtype=torch.bfloat16)
    lens = [90, 33, 150, 61, 120, 47, 77]
    reqs = {f"q{i}": seeded_ids(n, cfg["vocab_size"], 300 + i) for i, n in enumerate(lens)}
    steps, peak = rl.mixed(reqs, seed=5)
    eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=peak, page_size=page, max_requests=4, fuse="all")
    mixer = eng.model.blocks[0].mixer
    assert mixer.rope_in_product and mixer.qkv.rope_fuses(3, mixer.hd)
    rl.poison(eng)
    got = rl.run_in_process(eng, steps)
    for rid, ids in reqs.items():
        rows = torch.stack([got[(rid, p)] for p in range(len(ids))])
        assert torch.isfinite(rows).all(), rid
        assert rel_err(rows, plain_logits(folder, ids)) < TOL_BF16, rid
    eng.cache.check()
