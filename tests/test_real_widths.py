"""The layer sizes of Qwen2.5-1.5B (hidden 1536, 12/2 heads of 128, intermediate 8960, vocabulary
151936, tied head, q/k/v bias) with two layers and random weights: whole, in portions and token by
token against the plain implementation, in float32 and bfloat16.  Sizes that the tiny models do not
reach: the tensor-core attention and products at their real shapes, a vocabulary that is no
multiple of anything convenient, rows wider than the default shared-memory limit."""
import pytest
import torch

import replay_lib as rl
from helpers import TOL_BF16, TOL_F32, follows_plain, make_model, plain_logits, rel_err, seeded_ids

pytestmark = pytest.mark.gpu

WIDE = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 1536, "num_attention_heads": 12, "num_key_value_heads": 2,
    "intermediate_size": 8960, "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "use_sliding_window": False, "max_position_embeddings": 32768,
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_widths_whole_portions_and_single_tokens(model_root, dtype):
    from beglin_b200 import Engine
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = make_model(model_root, "wide", seed=4, dtype=stored, config=WIDE, std=0.02, bias_std=0.02)
    ids = {"a": seeded_ids(150, WIDE["vocab_size"], 1), "b": seeded_ids(70, WIDE["vocab_size"], 2)}
    want_rows = {"a": [0, 1, 63, 64, 149], "b": [0, 15, 16, 69]}
    want = {r: plain_logits(folder, ids[r]) for r in ids}
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=512, page_size=16, max_requests=4)
    rl.poison(eng)
    # whole, both requests in one step
    out = eng.step([("a", ids["a"], want_rows["a"]), ("b", ids["b"], want_rows["b"])], end=["a", "b"])
    got = {"a": out[:5], "b": out[5:]}
    for r in ids:
        assert rel_err(got[r], want[r][want_rows[r]]) < tol, r
    whole = out.clone()
    # in portions, the last tokens one by one, the two requests interleaved
    rows = []
    cuts = {"a": [0, 64, 129, 147, 148, 149, 150], "b": [0, 16, 17, 68, 69, 70]}
    keep = {"a": [], "b": []}
    for i in range(6):
        ents = []
        for r in ("a", "b"):
            c = cuts[r]
            if i + 1 < len(c):
                wanted = [p - c[i] for p in want_rows[r] if c[i] <= p < c[i + 1]]
                ents.append((r, ids[r][c[i]:c[i + 1]], wanted))
        out = eng.step(ents)
        row = 0
        for r, _, wanted in ents:
            if wanted:
                keep[r].append(out[row:row + len(wanted)])
                row += len(wanted)
    for r in ids:
        cut = torch.cat(keep[r])
        assert rel_err(cut, want[r][want_rows[r]]) < tol, r
    if dtype == "float32":
        assert torch.equal(torch.cat([torch.cat(keep["a"]), torch.cat(keep["b"])]), whole)
    # greedy decoding through the graph path agrees with the step function's logits
    eng.release("a"); eng.release("b")
    new = eng.generate([ids["b"][:20]], max_new_tokens=4, stop_ids=())[0]
    follows_plain(folder, ids["b"][:20], new, tol)


# The same widths with a vocabulary cut to 3,001 tokens, so that the float64 oracle runs six requests in
# seconds: the four ways of cutting of the replay tests, the mixed one on a pool so small that pages come back.
WIDE_SMALL_VOCAB = dict(WIDE, vocab_size=3001)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_widths_four_ways_of_cutting(model_root, dtype):
    """Each request alone and whole; most of it in one step and the last 32 tokens one by one; portions of
    changing size down to two tokens; and mixed, up to four live requests with portions of some beside single
    tokens of others, every page poisoned first.  float32: every row bitwise the same in the four ways (what a
    request computes does not depend on who shares its step, the reference's gate, qwen_infer.c:2040-2048, or
    on how it was cut) and right against the oracle; bfloat16: right against the oracle."""
    from beglin_b200 import Engine
    from test_replay import check_against_plain
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = make_model(model_root, "wide3001", seed=6, dtype=stored, config=WIDE_SMALL_VOCAB, std=0.02, bias_std=0.02)
    reqs = {f"r{i}": seeded_ids(n, 3001, 300 + i) for i, n in enumerate([150, 41, 290, 97, 64, 200])}
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    mixed_steps, peak = rl.mixed(reqs, seed=8)
    assert peak < sum(-(-len(v) // 64) * 64 for v in reqs.values())       # the pool cannot hold all at once
    results = {}
    for way, steps, max_tokens in (("whole", rl.whole(reqs), 320), ("tail", rl.last_one_by_one(reqs), 320),
                                   ("portions", rl.portions(reqs), 320), ("mixed", mixed_steps, peak)):
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, page_size=16, max_requests=4)
        rl.poison(eng)
        got = rl.run_in_process(eng, steps)
        eng.cache.check()
        assert eng.cache.free_pages() == eng.cache.num_pages and not eng.cache.live()
        worst = check_against_plain(got, folder, reqs, tol)
        print(f"real widths {dtype} {way}: worst relative error {worst:.3g} (limit {tol:g})")
        results[way] = got
        del eng
    if dtype == "float32":
        for way in ("tail", "portions", "mixed"):
            for key, row in results["whole"].items():
                assert torch.equal(row, results[way][key]), (way, key)
