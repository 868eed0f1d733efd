"""Seeded random configurations of the architecture: head counts and groups from 1 to 17 heads per kv head,
head sizes in steps of 16 up to 256, widths, intermediate sizes and vocabularies that are odd or no
multiple of anything, with and without a window, tied and untied, a head size given apart from
hidden / heads.  Each runs a mixed replay (up to four live requests, portions beside single tokens, a pool
so small that pages come back, every page poisoned first) in float32 or bfloat16 against the plain
implementation.  What the tiny test configurations pin by hand this covers broadly: a kernel either takes
a size or the engine picks another kernel for it; no size gives a wrong result."""
import random

import pytest
import torch

import replay_lib as rl
from helpers import TOL_BF16, TOL_F32, make_model, plain_logits, rel_err, seeded_ids

pytestmark = pytest.mark.gpu


def random_config(case):
    rng = random.Random(1234 + case)
    nkv = rng.choice([1, 1, 2, 3, 4])
    nh = nkv * rng.choice([1, 2, 3, 4, 6, 7, 8, 9, 16, 17])
    hd = rng.choice([16, 32, 48, 64, 64, 80, 96, 112, 128, 128, 144, 192, 256])
    hidden = rng.choice([nh * hd, rng.randrange(24, 400, 2), rng.randrange(24, 400, 8), rng.randrange(24, 300)])
    inter = rng.choice([rng.randrange(8, 500), 64 * rng.randrange(1, 8), 8 * rng.randrange(1, 60)])
    vocab = rng.choice([rng.randrange(50, 3000), 64 * rng.randrange(1, 40) + 1, 1000])
    cfg = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
           "num_hidden_layers": rng.choice([1, 2, 3]), "hidden_size": hidden, "num_attention_heads": nh,
           "num_key_value_heads": nkv, "head_dim": hd, "intermediate_size": inter, "vocab_size": vocab,
           "rope_theta": rng.choice([10000.0, 1e6, 500000.0]), "rms_norm_eps": rng.choice([1e-6, 1e-5, 1e-3]),
           "tie_word_embeddings": rng.random() < 0.5, "max_position_embeddings": 1024}
    if rng.random() < 0.3:
        cfg.update(use_sliding_window=True, sliding_window=rng.choice([5, 24, 64, 100]),
                   max_window_layers=rng.choice([0, 1]))
    if hidden == nh * hd and rng.random() < 0.5:
        del cfg["head_dim"]
    dtype = rng.choice(["float32", "bfloat16"])
    page = rng.choice([4, 8, 16, 32, 64])
    lens = [rng.randint(2, 300) for _ in range(5)]
    # weights small enough that the scores stay of order one at every width (a wide model with large
    # weights has a softmax so sharp that rounding alone moves the logits by more than the tolerance)
    std = min(0.05, 1.0 / max(hidden, nh * hd) ** 0.5)
    return cfg, dtype, page, lens, std


@pytest.mark.parametrize("case", range(32))
def test_random_configuration_mixed_replay(model_root, case):
    from beglin_b200 import Engine
    cfg, dtype, page, lens, std = random_config(case)
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = make_model(model_root, f"random{case}", seed=case, dtype=stored, config=cfg, std=std, bias_std=0.05)
    reqs = {f"q{i}": seeded_ids(n, cfg["vocab_size"], 1000 * case + i) for i, n in enumerate(lens)}
    steps, peak = rl.mixed(reqs, seed=case + 50)
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=peak, page_size=page, max_requests=4)
    rl.poison(eng)
    got = rl.run_in_process(eng, steps)
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    for rid, ids in reqs.items():
        rows = torch.stack([got[(rid, p)] for p in range(len(ids))])
        assert torch.isfinite(rows).all(), (rid, cfg)
        assert rel_err(rows, plain_logits(folder, ids)) < tol, (rid, cfg, dtype, page)
    eng.cache.check()


@pytest.mark.parametrize("case", [1, 3, 7, 12, 270, 526, 537, 565])
def test_random_configuration_prompts_then_single_tokens(model_root, case):
    """Several prompts whole in one step, then steps in which every request brings one token: through the step
    function and through `Engine.decode` (the replayed graph), both against the plain implementation.  Cases 270
    and 526 have q/k/v rows wider than 48 KB in float32; 537 has an intermediate size that the tcgen05 product
    does not take (no multiple of 8), so the library product runs inside the graph."""
    from beglin_b200 import Engine
    cfg, dtype, page, _, std = random_config(case)
    rng = random.Random(99 + case)
    n_req, n_dec = rng.choice([1, 2, 3, 5, 8]), rng.choice([8, 20, 40])
    prompt = [rng.randint(1, 200) for _ in range(n_req)]
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    folder = make_model(model_root, f"random{case}", seed=case, dtype=stored, config=cfg, std=std, bias_std=0.05)
    ids = [seeded_ids(p + n_dec, cfg["vocab_size"], 1000 * case + i) for i, p in enumerate(prompt)]
    want = [plain_logits(folder, x) for x in ids]
    for through_graph in (False, True):
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=sum(-(-len(x) // 64) * 64 for x in ids),
                                 page_size=page, max_requests=n_req)
        rl.poison(eng)
        out = eng.step([(i, ids[i][:prompt[i]], [prompt[i] - 1]) for i in range(n_req)])
        for i in range(n_req):
            assert rel_err(out[i:i + 1], want[i][[prompt[i] - 1]]) < tol, (case, "prompt", i)
        for k in range(n_dec):
            tokens = [ids[i][prompt[i] + k] for i in range(n_req)]
            if through_graph:
                eng.decode(list(range(n_req)), tokens, read_back=True)
                out = eng.decode_graph(n_req).logits
            else:
                out = eng.step([(i, [tokens[i]], [0]) for i in range(n_req)])
            assert torch.isfinite(out).all()
            for i in range(n_req):
                assert rel_err(out[i:i + 1], want[i][[prompt[i] + k]]) < tol, (case, through_graph, k, i)
        eng.cache.check()
