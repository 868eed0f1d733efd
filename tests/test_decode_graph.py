"""Decoding through the replayed graph in the shape that is benchmarked, and what the graph remembers.

The benchmark decodes through `Engine.decode`: one CUDA graph per batch size whose attention kernels are
launched for the context limit (4096), with requests of very different lengths side by side, the host
making room for the next step while the device runs this one.  Here that schedule is run at the benchmark's
head geometry (12 query heads on 2 kv heads of 128, pages of 64 and of 16) on a model narrow enough for the
float64 oracle: requests that hold 40, 700, 1,500 and 4,000 positions in ONE batch (so for the short ones
most CTAs of the fixed grid have no keys, and a growing request's keys cross the edges of pages and of key
ranges), 70 steps, teacher-forced so that every step's logits can be compared with the plain implementation,
and in float32 bitwise with the step function.

Also here: a request that ends and starts again under the same name at the same length (the graph must not
take it for the old one), batches that shrink through the graph sizes, and a mixer with state of its own
under graphs (the warm-up before a capture must not advance the state twice)."""
from dataclasses import dataclass

import pytest
import torch

import replay_lib as rl
from helpers import (TINY_B, TOL_BF16, TOL_F32, follows_plain, make_model, plain, plain_model, rel_err,
                     seeded_ids)

pytestmark = pytest.mark.gpu

# the benchmark's heads and pages on a narrow model: hidden 768 with head_dim given apart from it
GEOMETRY = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 768, "num_attention_heads": 12, "num_key_value_heads": 2, "head_dim": 128,
    "intermediate_size": 1536, "vocab_size": 1000, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "use_sliding_window": False, "max_position_embeddings": 32768,
}
STEPS = 70
LENGTHS_8 = [40, 700, 1500, 4000, 63, 1023, 255, 2049]
# 64 requests: the four of the benchmark's spread first, then lengths at and around the edges of pages (64) and
# of the decoding kernel's key stages (256)
LENGTHS_64 = [40, 700, 1500, 4000] + [1 + (37 * i * i + 11 * i) % 900 for i in range(52)] + \
             [63, 64, 65, 255, 256, 257, 1023, 1024]


def oracle_rows(folder, ids, first):
    """float64 logits of rows first.. of the whole sequence, computed on the GPU by the plain implementation."""
    cfg, w = plain_model(folder)
    key = ("cuda", folder)
    from helpers import _PLAIN_CACHE
    if key not in _PLAIN_CACHE:
        _PLAIN_CACHE[key] = {k: v.cuda() for k, v in w.items()}
    return plain.forward(cfg, _PLAIN_CACHE[key], list(ids))[first:].cpu()


def fill(eng, ids, lengths, chunk=1024):
    """Prompts through the step function, several requests a step, portions of `chunk`."""
    pending = list(range(len(lengths)))
    while pending:
        group = []
        while pending and len(group) < 8:
            group.append(pending.pop(0))
        longest = max(lengths[i] for i in group)
        for lo in range(0, longest, chunk):
            ents = [(i, ids[i][lo:min(lengths[i], lo + chunk)], []) for i in group if lo < lengths[i]]
            eng.step(ents, check=False)


@pytest.mark.parametrize("dtype,page,lengths", [("float32", 64, LENGTHS_8), ("bfloat16", 64, LENGTHS_8),
                                                ("bfloat16", 16, LENGTHS_8), ("float32", 16, LENGTHS_8),
                                                ("bfloat16", 64, LENGTHS_64), ("float32", 64, LENGTHS_64)])
def test_graph_decoding_at_the_benchmark_geometry(model_root, dtype, page, lengths):
    from beglin_b200 import Engine
    from beglin_b200.csrc import ops
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = make_model(model_root, "geometry", seed=31, dtype=stored, config=GEOMETRY, std=0.03, bias_std=0.05)
    n = len(lengths)
    ids = [seeded_ids(L + STEPS, GEOMETRY["vocab_size"], 500 + i) for i, L in enumerate(lengths)]
    want = [oracle_rows(folder, ids[i], lengths[i]) for i in range(n)]           # [STEPS, vocab] each
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    pool = sum(-(-(L + STEPS) // 64) * 64 for L in lengths)
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=pool, page_size=page, max_requests=n, max_context=4096)
    rl.poison(eng)
    fill(eng, ids, lengths)
    rids = list(range(n))
    g = eng.decode_graph(n)
    assert g.batch.max_position == 4095                       # the grid is laid out for the context limit
    worst, ahead = 0.0, 0
    graph_rows = []
    for k in range(STEPS):
        ahead += int(g.prepared(rids))
        eng.decode(rids, [ids[i][lengths[i] + k] for i in range(n)], read_back=True)
        out = g.logits[:n].float().cpu()
        assert torch.isfinite(out).all(), k
        graph_rows.append(out)
        for i in range(n):
            err = rel_err(out[i:i + 1], want[i][k:k + 1])
            worst = max(worst, err)
            assert err < tol, (dtype, page, "step", k, "request", i, "length", lengths[i] + k, err)
    assert ahead >= STEPS - 2                                 # the host had made room ahead of nearly every step
    ops.raise_on_status(eng.ctx.status)
    eng.cache.check()
    if dtype == "float32":
        # the same steps through the step function, kernel by kernel, from a fresh cache: bitwise the same rows
        for r in rids:
            eng.release(r)
        rl.poison(eng)
        fill(eng, ids, lengths)
        for k in range(STEPS):
            out = eng.step([(i, [ids[i][lengths[i] + k]], [0]) for i in range(n)], check=False).cpu()
            assert torch.equal(out, graph_rows[k]), k
    print(f"graph decoding {dtype} page {page} batch {n}: worst relative error {worst:.2e}")


def test_a_request_that_starts_again_under_its_name_at_the_same_length(model_root):
    """`generate` names its requests by their index.  A second call whose first decoding step has the same names
    and the same lengths as the first call's last remembered step must not be taken for it: its pages are
    others.  Five tokens, eight new ones; then a prompt of twelve that decodes from length 12 = 5 + 8 - 1."""
    from beglin_b200 import Engine
    folder = make_model(model_root, "A", seed=3, dtype=torch.float32)
    cfg, w = plain_model(folder)
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=512, page_size=8, max_requests=4)
    first, other, second = seeded_ids(5, 256, 1), seeded_ids(29, 256, 9), seeded_ids(12, 256, 2)
    assert eng.generate([first], max_new_tokens=8, stop_ids=()) == [plain.greedy_generate(cfg, w, first, 8)]
    # pages change hands in between (two prompts that end with their first token: no decoding step, so the graph
    # still remembers the first call's last step), and the restarted name finds its pages elsewhere
    assert eng.generate([other, second], max_new_tokens=[1, 1], stop_ids=())[0] == plain.greedy_generate(cfg, w, other, 1)
    assert eng.generate([second], max_new_tokens=6, stop_ids=()) == [plain.greedy_generate(cfg, w, second, 6)]
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batches_that_shrink_go_through_few_graphs(model_root, dtype):
    """Six requests with token limits 3..18 end one by one: the decoding steps run batches of 6, 5, ... 1
    through the graphs of 8, 4, 2 and 1 rows, the spare rows writing to the spare page.  float32: the tokens of
    the plain implementation.  bfloat16: teacher-forced, every token within the rounding of its row's maximum."""
    from beglin_b200 import Engine
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = make_model(model_root, "D", seed=17, dtype=stored)
    cfg, w = plain_model(folder)
    prompts = [seeded_ids(n, 200, 40 + n) for n in (9, 30, 17, 70, 5, 64)]
    limits = [3, 6, 9, 12, 15, 18]
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024, page_size=16, max_requests=6)
    rl.poison(eng)
    outs = eng.generate(prompts, max_new_tokens=limits, stop_ids=())
    assert sorted(eng._graphs) == [1, 2, 4, 8]
    assert [len(o) for o in outs] == limits
    for p, out in zip(prompts, outs):
        if dtype == "float32":
            assert out == plain.greedy_generate(cfg, w, p, len(out))
        else:
            follows_plain(folder, p, out)
    eng.cache.check()
    assert eng.cache.free_pages() == eng.cache.num_pages


# ------------------------------------------------------------------------------------------------
# A mixer with state of its own whose forward is fit for stream capture: state <- decay * state + W h_t.

@dataclass(frozen=True)
class CapturableDecaySpec:
    hidden: int
    decay: float
    kind: str = "toy_decay_capturable"


def register_capturable_decay():
    from beglin_b200.parts import FixedStateNeed, Linear, TensorRole, register_mixer

    @register_mixer("toy_decay_capturable")
    class CapturableDecay:
        @staticmethod
        def expected_tensors(spec):
            return [TensorRole("w.weight", (spec.hidden, spec.hidden), True, True)]

        @staticmethod
        def cache_need(spec):
            return FixedStateNeed((spec.hidden,), "float32")

        def __init__(self, spec, tensors, ctx):
            self.spec, self.ctx = spec, ctx
            self.w = Linear(tensors["w.weight"], None, ctx)

        def forward(self, h, batch, cache):
            """Only sizes of the batch are used on the host (row_start, lens); the slots stay on the device."""
            u = self.w(h).float()
            out = torch.empty_like(u)
            slots = cache.slots.long()
            for i, (r0, n) in enumerate(zip(batch.row_start, batch.lens)):
                s = cache.state.index_select(0, slots[i:i + 1])[0]
                for t in range(r0, r0 + n):
                    s = s * self.spec.decay + u[t]
                    out[t] = s
                cache.state.index_copy_(0, slots[i:i + 1], s[None])
            return out.to(self.ctx.compute_dtype)

    return CapturableDecay


def test_state_of_fixed_size_under_graphs():
    """Layer 1 of three carries a state vector per request.  Decoding steps are replayed as graphs (the step that
    captures a graph runs its body twice: once to warm up, once as the replay) and so is a repeated portion; the
    state must advance once per token all the same.  Compared with the plain computation."""
    from beglin_b200 import Engine
    from beglin_b200.config import load_config
    from beglin_b200.weights import TensorDict, random_tensors
    import test_parts
    register_capturable_decay()
    arch, cfg = load_config(TINY_B)
    spec = arch.build_spec(cfg)
    l1 = spec.layers[1]
    names = {k: v for k, v in l1.names.items() if not k.startswith("mixer.")}
    names["mixer.w.weight"] = "model.layers.1.toy.w.weight"
    spec.layers[1] = l1.with_parts(mixer=CapturableDecaySpec(hidden=cfg.hidden_size, decay=0.5), names=names)
    tensors = random_tensors(spec, 5, std=0.05, dtype=torch.float32)
    eng = Engine(spec, TensorDict(tensors), dtype="float32", max_tokens=512, page_size=16, max_requests=3, kv_split=64,
                 portion_graph_rows=16)
    w = {k: v.double() for k, v in tensors.items()}
    ids = {"a": seeded_ids(60, 384, 1), "b": seeded_ids(41, 384, 2), "c": seeded_ids(25, 384, 3)}
    start = {"a": 30, "b": 11, "c": 5}
    want = {r: test_parts.plain_toy_forward(TINY_B, w, ids[r], [0, 1, 2], False) for r in ids}
    # prompts, then decoding through the graph of four rows (three requests and a spare row, whose state goes
    # to the spare slot): the first decoding step captures
    out = eng.step([(r, ids[r][:start[r]], [start[r] - 1]) for r in "abc"])
    for i, r in enumerate("abc"):
        assert rel_err(out[i:i + 1], want[r][start[r] - 1:start[r]]) < 1e-4
    for k in range(10):
        eng.decode(list("abc"), [ids[r][start[r] + k] for r in "abc"])
        out = eng.decode_graph(3).logits
        assert out.shape[0] == 4
        for i, r in enumerate("abc"):
            assert rel_err(out[i:i + 1], want[r][start[r] + k:start[r] + k + 1]) < 1e-4, (k, r)
    # one request alone (another graph, captured on this step), then portions of 20 tokens of a new request: the
    # second portion of that shape captures a portion graph, the third replays it
    eng.decode(["b"], [ids["b"][21]])
    assert rel_err(eng.decode_graph(1).logits[0:1], want["b"][21:22]) < 1e-4
    for r in "abc":
        eng.release(r)
    got = [eng.step([("d", ids["a"][lo:lo + 20], [19])]) for lo in (0, 20, 40)]
    assert eng.portions.replays >= 2
    assert rel_err(torch.cat(got), want["a"][[19, 39, 59]]) < 1e-4
