"""Traces for the replay tests: the same requests whole, with the last 32 tokens one by one, in
portions of changing size, and mixed with other requests on a pool so small that pages are reused."""
import random
from typing import Dict, List

import torch


def whole(reqs: Dict[str, List[int]]):
    steps = []
    for rid, ids in reqs.items():
        steps.append({"entries": [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}], "end": [rid]})
    return steps


def last_one_by_one(reqs, tail=32):
    steps = []
    for rid, ids in reqs.items():
        head = len(ids) - tail
        assert head >= 1
        steps.append({"entries": [{"id": rid, "tokens": ids[:head], "want": list(range(head))}], "end": []})
        for i in range(head, len(ids)):
            steps.append({"entries": [{"id": rid, "tokens": [ids[i]], "want": [0]}],
                          "end": [rid] if i == len(ids) - 1 else []})
    return steps


def portions(reqs, sizes=(16, 7, 4, 3, 2, 2, 5, 9, 2, 31, 1, 6)):
    steps = []
    for k, (rid, ids) in enumerate(reqs.items()):
        pos, i = 0, k
        while pos < len(ids):
            n = min(sizes[i % len(sizes)], len(ids) - pos)
            if len(ids) - pos - n == 1:          # never leave a lone last token: portions go down to two
                n += 1
            steps.append({"entries": [{"id": rid, "tokens": ids[pos:pos + n], "want": list(range(n))}],
                          "end": [rid] if pos + n == len(ids) else []})
            pos += n
            i += 1
    return steps


def mixed(reqs, seed=0, max_live=4):
    """Up to `max_live` requests at a time; each step takes a portion of some (sometimes a single
    token, like a decoded one) and leaves others out.  Returns (steps, max_tokens) where max_tokens
    is the most the live requests ever hold, each rounded up to 64."""
    rng = random.Random(seed)
    waiting = list(reqs.items())
    live: Dict[str, int] = {}
    steps = []
    peak = 0
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.7):
            rid, _ = waiting.pop(0)
            live[rid] = 0
        entries, end = [], []
        for rid in list(live):
            if len(live) > 1 and rng.random() < 0.25:
                continue                                        # left out of this step, goes on later
            ids = reqs[rid]
            left = len(ids) - live[rid]
            r = rng.random()
            n = 1 if r < 0.4 else rng.choice([2, 2, 3, 5, 8, 13, 17, 30])
            n = min(n, left)
            entries.append({"id": rid, "tokens": ids[live[rid]:live[rid] + n], "want": list(range(n))})
            live[rid] += n
        peak = max(peak, sum(-(-n // 64) * 64 for n in live.values()))
        for rid in list(live):
            if live[rid] == len(reqs[rid]):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append({"entries": entries, "end": end})
    return steps, peak


def number(steps):
    return [dict(s, step=i) for i, s in enumerate(steps)]


def run_in_process(engine, steps):
    """Feed the steps to Engine.step; returns {(request, position): float32 logits row on the CPU}."""
    out = {}
    held: Dict[str, int] = {}
    for s in steps:
        logits = engine.step(s["entries"], end=s.get("end", []))
        row = 0
        for e in s["entries"]:
            start = held.get(e["id"], 0)
            for w in e["want"]:
                out[(e["id"], start + w)] = logits[row].float().cpu()
                row += 1
            held[e["id"]] = start + len(e["tokens"])
        assert (0 if logits is None else logits.shape[0]) == row
        for rid in s.get("end", []):
            held.pop(rid, None)
    return out


def poison(engine):
    """Fill every page with NaN so that a read of a page that was never written shows."""
    for g in engine.cache.kv_groups:
        g.device_pool.fill_(float("nan"))
