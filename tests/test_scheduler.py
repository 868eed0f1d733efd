"""The scheduler's decisions (no GPU): admission order, decode rows first, portions under a token
budget, endings, and what happens when pages run out.  A fake step stands in for the model: the
token it "samples" depends only on the request's tokens so far, so recomputation after a preemption
must reproduce the same output."""
import zlib

import pytest

from beglin_b200.cache import CacheManager
from beglin_b200.engine.scheduler import Request, Scheduler
from beglin_b200.parts.cache_need import PagedKVNeed


def fake_token(history):
    return zlib.crc32(repr(list(history)).encode()) % 1000


def run(sched, reqs, max_steps=10000, on_step=None):
    for r in reqs:
        sched.add(r)
    held = {}                                        # request -> tokens fed so far (mirrors the cache)
    steps = []
    for _ in range(max_steps):
        plan = sched.plan()
        if plan is None:
            break
        sched.cache.check()
        for e in plan.entries:
            start = sched.cache.length(e.rid)
            hist = held.get(e.rid, [])
            hist = hist[:start] + list(e.tokens)     # a preempted request starts again from 0
            held[e.rid] = hist
            assert sched.cache.pages_held(e.rid) * sched.cache.page_size >= len(hist)
        wanted = sched.wanted(plan)
        toks = [fake_token(held[r.rid]) for r in wanted]
        steps.append(plan)
        if on_step:
            on_step(plan)
        sched.update(plan, toks)
        sched.cache.check()
    else:
        raise AssertionError("scheduler did not finish")
    return steps


def cache(pages=64, page=4, reqs=8, ctx=None):
    return CacheManager([PagedKVNeed(1, 16)], page_size=page, num_pages=pages, max_requests=reqs, max_context=ctx)


def expected_output(prompt, n, stop=()):
    hist, out = list(prompt), []
    for _ in range(n):
        t = fake_token(hist)
        out.append(t); hist.append(t)
        if t in stop:
            break
    return out


def test_fifo_admission_decode_first_and_budget():
    c = cache()
    s = Scheduler(c, max_batch=2, max_step_tokens=8)
    reqs = [Request(i, list(range(10 + i, 10 + i + n)), m) for i, (n, m) in enumerate([(11, 6), (5, 2), (3, 3)])]
    steps = run(s, reqs)
    # first step: budget 8 all to request 0 (slot order), request 1 admitted but waits for budget
    assert [(e.rid, len(e.tokens)) for e in steps[0].entries] == [(0, 8)]
    assert [(e.rid, len(e.tokens)) for e in steps[1].entries] == [(0, 3), (1, 5)]
    assert steps[1].entries[0].want == [2] and steps[1].entries[1].want == [4]
    # once decoding, a request's single token comes before any prompt portion
    for p in steps:
        kinds = [len(e.tokens) == 1 and e.rid in [r.rid for r in p.decode] for e in p.entries]
        assert kinds == sorted(kinds, reverse=True)
        assert p.n_tokens <= 8
    # request 2 is admitted only after a slot is free
    first2 = next(i for i, p in enumerate(steps) if any(e.rid == 2 for e in p.entries))
    done_before = [r for r in (reqs[0], reqs[1]) if r.finish_reason]
    assert first2 > 1 and done_before
    for r in reqs:
        assert r.output == expected_output(r.prompt, r.max_new_tokens) and r.finish_reason == "length"
    assert c.free_pages() == 64 and not c.live()
    assert s.counters.mixed_steps >= 1 and s.counters.steps == len(steps)


def test_prefill_budget_option():
    c = cache()
    s = Scheduler(c, max_batch=4, max_step_tokens=64, prefill_budget=3)
    reqs = [Request("a", list(range(7)), 2), Request("b", list(range(5)), 2)]
    steps = run(s, reqs)
    assert [(e.rid, len(e.tokens)) for e in steps[0].entries] == [("a", 3)]
    assert [(e.rid, len(e.tokens)) for e in steps[2].entries] == [("a", 1), ("b", 2)]
    assert all(sum(len(e.tokens) for e in p.entries if len(e.tokens) > 1 or e.rid not in [r.rid for r in p.decode]) <= 3
               for p in steps)


def test_stop_token_is_recorded_and_ends_the_request():
    c = cache()
    prompt = [5, 6, 7]
    full = expected_output(prompt, 6)
    stop = full[2]
    s = Scheduler(c)
    r = Request("x", prompt, 6, stop_ids=(stop,))
    run(s, [r])
    assert r.output == full[:3] and r.finish_reason == "stop"


def test_context_limit_ends_generation():
    c = cache(ctx=8)
    s = Scheduler(c)
    r = Request("x", [1, 2, 3, 4, 5], 10)
    run(s, [r])
    # positions 0..7 can be held: 5 prompt + 3 generated tokens fed; the 4th token is sampled but cannot be fed
    assert r.finish_reason == "context_limit" and len(r.output) == 4
    r2 = Request("y", list(range(8)), 4)
    s2 = Scheduler(cache(ctx=8))
    run(s2, [r2])
    assert r2.finish_reason == "context_limit" and r2.output == []


def test_out_of_pages_preempts_last_admitted_and_recomputes():
    c = cache(pages=6, page=4)                    # 24 positions in all
    s = Scheduler(c, max_batch=3, max_step_tokens=64)
    reqs = [Request("a", list(range(8)), 12), Request("b", list(range(20, 27)), 12)]
    preempted = []
    steps = run(s, reqs)
    assert s.counters.preemptions >= 1
    assert reqs[1].preemptions >= 1 and reqs[0].preemptions == 0          # the one admitted last yields
    for r in reqs:
        assert r.output == expected_output(r.prompt, 12), r.rid
        assert r.finish_reason == "length"
    assert c.free_pages() == 6


def test_request_that_cannot_fit_alone_ends_with_out_of_pages():
    c = cache(pages=2, page=4, ctx=64)
    s = Scheduler(c, max_step_tokens=64)
    big = Request("big", list(range(6)), 20)
    small = Request("small", [1, 2], 3)
    run(s, [big, small])
    assert big.finish_reason == "out_of_pages" and len(big.output) >= 1
    assert small.finish_reason == "length" and small.output == expected_output([1, 2], 3)
    assert c.free_pages() == 2


def test_prompt_portions_shrink_to_the_free_pages():
    c = cache(pages=4, page=4, ctx=64)
    s = Scheduler(c, max_batch=2, max_step_tokens=64)
    a = Request("a", list(range(9)), 2)            # 3 pages
    b = Request("b", list(range(30, 36)), 2)       # would need 2 pages; only 1 is free at first
    steps = run(s, [a, b])
    assert [(e.rid, len(e.tokens)) for e in steps[0].entries] == [("a", 9), ("b", 4)]
    assert a.output == expected_output(a.prompt, 2) and b.output == expected_output(b.prompt, 2)


def test_repeats_are_identical():
    outs = []
    for _ in range(2):
        c = cache(pages=10, page=4)
        s = Scheduler(c, max_batch=3, max_step_tokens=16)
        reqs = [Request(i, list(range(i, i + 3 + 2 * i)), 5 + i) for i in range(5)]
        steps = run(s, reqs)
        outs.append(([r.output for r in reqs], [[(e.rid, tuple(e.tokens)) for e in p.entries] for p in steps]))
    assert outs[0] == outs[1]


def test_inter_token_gaps_and_utilisation_are_counted_as_the_reference_counts_them():
    """One clock reading per step; a request's gap runs from the step that gave its previous token to the
    step that gives the next one, its first token starting the clock; a request that waits while another's
    prompt runs alone shows a longer gap (qwen_infer.c:20731-20742)."""
    ticks = iter(range(1000))
    c = cache()
    s = Scheduler(c, max_batch=2, max_step_tokens=64, prefill_budget=4, now=lambda: float(next(ticks)))
    reqs = [Request(0, [1, 2, 3], 4), Request(1, list(range(20, 28)), 2)]
    steps = run(s, reqs)
    # step 0: request 0 whole (3 tokens) and the first token of request 1's prompt (budget 4); request 0 then
    # decodes in every step, so its three gaps are one tick each; request 1 needs two more steps of prompt,
    # gets its first token at the end of step 2 and its second one step later: one gap of one tick
    assert [[(e.rid, len(e.tokens)) for e in p.entries] for p in steps[:3]] == [[(0, 3), (1, 1)], [(0, 1), (1, 4)], [(0, 1), (1, 3)]]
    k = s.counters
    assert k.gaps == 3 + 1 and k.gap_max_s == 1.0 and k.gap_mean_s() == 1.0
    assert k.steps == len(steps) == 4 and k.decode_rows == 3 + 1
    assert k.utilisation(2) == 4 / (4 * 2)
    assert reqs[0].output == expected_output([1, 2, 3], 4) and reqs[1].output == expected_output(range(20, 28), 2)


def test_a_preempted_request_shows_its_recomputation_as_a_gap():
    ticks = iter(range(1000))
    c = cache(pages=5, page=4, reqs=4)
    s = Scheduler(c, max_batch=2, max_step_tokens=64, now=lambda: float(next(ticks)))
    reqs = [Request(0, list(range(7)), 12), Request(1, list(range(50, 57)), 6)]
    run(s, reqs)
    assert s.counters.preemptions >= 1
    assert s.counters.gap_max_s > 1.0                     # the victim's next token came more than a step later
    assert s.counters.gaps == (12 - 1) + (6 - 1)          # every token but a request's first closes a gap


def test_sequential_prefill_gives_the_same_tokens_and_shows_the_stalls():
    """QWEN_CB_MIXED=0, the reference's older order (qwen_infer.c:20759-20782): a request's whole prompt runs in
    steps of its own while the decoding requests wait.  Every request gets the tokens it gets in the mixed
    order (the reference's gate, qwen_infer.c:20641-20645); what differs is what the counters show: steps in
    which decoding stalled, no mixed steps, and a longer worst gap between a request's tokens."""
    def workload():
        return [Request(i, list(range(100 * i, 100 * i + n)), m) for i, (n, m) in
                enumerate([(5, 9), (23, 4), (3, 12), (40, 3), (9, 6), (17, 5)])]
    results = {}
    for mixed in (True, False):
        ticks = iter(range(100000))
        s = Scheduler(cache(), max_batch=3, max_step_tokens=64, prefill_budget=8, mixed=mixed, now=lambda: float(next(ticks)))
        reqs = workload()
        steps = run(s, reqs)
        for r in reqs:
            assert r.output == expected_output(r.prompt, r.max_new_tokens) and r.finish_reason == "length"
        results[mixed] = (s.counters, steps, [r.output for r in reqs])
    assert results[True][2] == results[False][2]
    mixed_c, seq_c = results[True][0], results[False][0]
    assert mixed_c.mixed_steps > 0 and mixed_c.prefill_stalls == 0
    assert seq_c.mixed_steps == 0 and seq_c.prefill_stalls > 0
    assert seq_c.gap_max_s > mixed_c.gap_max_s                # a 40-token prompt in portions of 8 holds the decoders up
    for p in results[False][1]:                               # a step is either one request's portion or decoding rows
        kinds = {len(e.tokens) == 1 and e.rid in [r.rid for r in p.decode] for e in p.entries}
        assert len(kinds) == 1 and (kinds == {True} or len(p.entries) == 1)
        assert p.n_tokens <= 8 or all(len(e.tokens) == 1 for e in p.entries)


def test_sequential_prefill_with_few_pages_still_ends():
    """When no portion fits beside the room the waiting decoders need, they decode after all; nobody starves."""
    s = Scheduler(cache(pages=7, page=4), max_batch=3, max_step_tokens=64, prefill_budget=8, mixed=False)
    reqs = [Request("a", list(range(8)), 10), Request("b", list(range(20, 31)), 6), Request("c", list(range(40, 45)), 4)]
    run(s, reqs)
    for r in reqs:
        assert r.output == expected_output(r.prompt, r.max_new_tokens), r.rid
    assert s.cache.free_pages() == 7
