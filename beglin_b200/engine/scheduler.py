"""The scheduler above the step function.

It follows the reference's mixed continuous-batching loop (qwen_infer.c:20803-20853): requests wait
in a FIFO queue; a free slot is taken at once, without forward work; every step carries one token
of every decoding request first, then prompt portions of the requests still in prefill, in slot
order, under a token budget; the last prompt token's logits give the first new token; a request
ends on a stop token (which is recorded), on its token limit, or at the context limit
(qwen_infer.c:20840).

The reference's cache is static, so it cannot run out.  Pages can.  The decision here: decoding
rows always come first; if their next positions need more pages than are free, the request admitted
LAST is preempted: it gives back all it holds and returns to the head of the queue with the tokens it
has generated appended to its prompt, to be recomputed when admitted again.  Prompt portions are
shortened to what the free pages hold, down to nothing.  A request that does not fit even when it is
the only one ends with the reason "out_of_pages".

Pure host code: it talks to the cache manager's accounting and is tested without a GPU.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence, Set, Tuple

from ..cache.manager import CacheManager
from .batch import Entry


@dataclass
class Request:
    rid: Hashable
    prompt: List[int]
    max_new_tokens: int
    temperature: float = 0.0
    seed: int = 0
    stop_ids: Tuple[int, ...] = ()
    # filled by the scheduler
    output: List[int] = field(default_factory=list)
    phase: str = "waiting"            # waiting, prefill, decode, done
    done_prompt: int = 0              # prompt tokens already in the cache (of `tokens_in`)
    tokens_in: List[int] = field(default_factory=list)   # what must be in the cache before decoding
    finish_reason: Optional[str] = None
    admitted_at: int = -1
    preemptions: int = 0
    last_token_at: Optional[float] = None     # when the step that gave its newest token was recorded


@dataclass
class StepPlan:
    entries: List[Entry]
    decode: List[Request]             # requests whose entry is one decoded token, in entry order
    prefill: List[Tuple[Request, int, bool]]   # (request, tokens taken, reaches the prompt's end)
    lengths: List[Tuple[Hashable, int]] = field(default_factory=list)   # (request, length after the step): what was reserved

    @property
    def n_tokens(self) -> int:
        return sum(len(e.tokens) for e in self.entries)


@dataclass
class Counters:
    steps: int = 0
    mixed_steps: int = 0
    prefill_only_steps: int = 0
    decode_rows: int = 0
    prefill_rows: int = 0
    preemptions: int = 0
    prefill_stalls: int = 0           # sequential prefill only: prompt steps that ran while decoding requests sat idle
    # time between consecutive tokens of one request, from its first token on (the reference's inter-token gap,
    # qwen_infer.c:20731-20742: taken once per step, so that a request which gets nothing while others' prompts
    # run, or which is recomputed after a preemption, shows as a long gap)
    gaps: int = 0
    gap_sum_s: float = 0.0
    gap_max_s: float = 0.0

    def utilisation(self, batch: int) -> float:
        """Decoding rows per step over the live-request limit (qwen_infer.c:20879)."""
        return self.decode_rows / (self.steps * batch) if self.steps and batch else 0.0

    def gap_mean_s(self) -> float:
        return self.gap_sum_s / self.gaps if self.gaps else 0.0


class Scheduler:
    def __init__(self, cache: CacheManager, max_batch: int = 8, max_step_tokens: int = 2048,
                 prefill_budget: Optional[int] = None, max_context: Optional[int] = None, now=time.perf_counter,
                 mixed: bool = True):
        """max_batch: live requests (the reference's QWEN_BATCH, default 8, qwen_infer.c:20617);
        prefill_budget: prompt tokens per step (QWEN_CB_PREFILL_BUDGET, qwen_infer.c:20691), by
        default whatever max_step_tokens leaves after the decoding rows.
        mixed (QWEN_CB_MIXED, qwen_infer.c:20690): True puts prompt portions beside the decoding rows of
        a step.  False is the reference's older order (qwen_infer.c:20759-20782): while any admitted request
        still has prompt left, a step carries ONE request's next portion and nothing else, and the decoding
        requests wait; it exists so that the two can be compared (worst gap between a request's tokens,
        steps in which decoding stalled), and both give every request the same tokens."""
        self.cache = cache
        self.mixed = mixed
        self.max_batch = min(max_batch, cache.max_requests)
        self.max_step_tokens = max_step_tokens
        self.prefill_budget = prefill_budget
        self.max_context = min(max_context or cache.max_context, cache.max_context)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []         # in slot order = admission order
        self.finished: List[Request] = []
        self.counters = Counters()
        self._clock = 0
        self._now = now                          # the clock of the inter-token gaps

    # ------------------------------------------------------------------ queue
    def add(self, req: Request) -> None:
        if not req.prompt:
            raise ValueError(f"request {req.rid!r} has an empty prompt")
        req.tokens_in = list(req.prompt)
        req.phase = "waiting"
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def _finish(self, req: Request, reason: str) -> None:
        req.phase, req.finish_reason = "done", reason
        if self.cache.has(req.rid):
            self.cache.release(req.rid)
        if req in self.running:
            self.running.remove(req)
        self.finished.append(req)

    def _preempt(self, req: Request) -> None:
        """Give back what `req` holds and queue it again, first in line, to be recomputed."""
        self.cache.release(req.rid)
        self.running.remove(req)
        req.tokens_in = list(req.prompt) + list(req.output)
        req.done_prompt = 0
        req.phase = "waiting"
        req.preemptions += 1
        self.counters.preemptions += 1
        self.waiting.appendleft(req)

    def _admit(self) -> None:
        while self.waiting and len(self.running) < self.max_batch and self.cache.can_add():
            req = self.waiting[0]
            if len(req.tokens_in) + 1 > self.max_context and not req.output:
                # the prompt alone fills the context: nothing can be generated (qwen_infer.c:20851)
                self.waiting.popleft()
                self.finished.append(req)
                req.phase, req.finish_reason = "done", "context_limit"
                continue
            if self.running and self.cache.free_pages() < 1:
                break                               # no room to make progress on another request
            self.waiting.popleft()
            self.cache.add_request(req.rid)
            req.phase = "prefill"
            req.admitted_at = self._clock
            self._clock += 1
            self.running.append(req)

    # ------------------------------------------------------------------ one step
    def plan(self) -> Optional[StepPlan]:
        """Decide the next step, reserve its pages, and return it; None when nothing is left."""
        while True:
            self._admit()
            if not self.running:
                if not self.waiting:
                    return None
                continue
            decode = [r for r in self.running if r.phase == "decode"]
            # decoding rows first; preempt the last admitted until their pages fit
            while decode:
                plan = [(r.rid, self.cache.length(r.rid) + 1) for r in decode]
                if self.cache.pages_short(plan) == 0:
                    break
                victim = max(self.running, key=lambda r: r.admitted_at)
                if len(self.running) == 1:
                    self._finish(victim, "out_of_pages")
                else:
                    self._preempt(victim)
                decode = [r for r in self.running if r.phase == "decode"]
            if not self.running:
                continue
            plan = [(r.rid, self.cache.length(r.rid) + 1) for r in decode]
            budget = self.max_step_tokens - len(decode)
            if self.prefill_budget is not None:
                budget = min(budget, self.prefill_budget)
            if not decode:
                budget = max(budget, 1)             # progress guarantee (qwen_infer.c:20815-20817)
            stalled: List[Request] = []
            if not self.mixed and any(r.phase == "prefill" for r in self.running):
                # sequential prefill: this step is one request's portion alone; the decoding requests keep
                # their pages (made sure of above) and wait
                stalled, decode, plan = decode, [], []
                budget = max(1, self.prefill_budget if self.prefill_budget is not None else self.max_step_tokens)
            prefill: List[Tuple[Request, int, bool]] = []
            for r in self.running:
                if r.phase != "prefill" or budget <= 0 or (prefill and not self.mixed):
                    continue
                have = self.cache.length(r.rid)
                take = min(len(r.tokens_in) - r.done_prompt, budget)
                held = [(q.rid, self.cache.length(q.rid) + 1) for q in stalled]     # room the waiting rows will need
                while take > 0 and self.cache.pages_short(held + plan + [(r.rid, have + take)]) > 0:
                    # give up the portion's last page: shorten it to the previous page boundary
                    take = ((have + take - 1) // self.cache.page_size) * self.cache.page_size - have
                if take <= 0:
                    continue
                plan.append((r.rid, have + take))
                prefill.append((r, take, r.done_prompt + take == len(r.tokens_in)))
                budget -= take
            if stalled and not prefill:
                # sequential order, and no portion fits beside the room the decoding requests need next: they
                # decode after all, and what they free when they end lets the prompt go on
                decode, stalled = stalled, []
                plan = [(r.rid, self.cache.length(r.rid) + 1) for r in decode]
            if not decode and not prefill:
                # nothing fits: free the pages of the request admitted last, or give up on the only one
                victim = max(self.running, key=lambda r: r.admitted_at)
                if len(self.running) == 1:
                    self._finish(victim, "out_of_pages")
                else:
                    self._preempt(victim)
                continue
            self.cache.reserve(plan)
            entries = [Entry(r.rid, [r.output[-1]], [0]) for r in decode]
            for r, take, last in prefill:
                toks = r.tokens_in[r.done_prompt:r.done_prompt + take]
                entries.append(Entry(r.rid, toks, [take - 1] if last else []))
            lengths = plan
            c = self.counters
            c.steps += 1
            c.decode_rows += len(decode)
            c.prefill_rows += sum(t for _, t, _ in prefill)
            if decode and prefill:
                c.mixed_steps += 1
            if not decode:
                c.prefill_only_steps += 1
            if stalled:
                c.prefill_stalls += 1
            return StepPlan(entries, decode, prefill, lengths)

    def wanted(self, plan: StepPlan) -> List[Request]:
        """The requests that get a new token from this step, in the order of the step's logit rows."""
        return list(plan.decode) + [r for r, _, last in plan.prefill if last]

    def update(self, plan: StepPlan, tokens: Sequence[int], committed: bool = False) -> List[Request]:
        """Record the step: new lengths (unless the step function that ran the plan has `committed` them to
        the cache already), the sampled token of every request in `wanted(plan)`, phase changes and endings.
        Returns the requests that ended."""
        if not committed:
            self.cache.commit(plan.lengths)
        for r, take, last in plan.prefill:
            r.done_prompt += take
        ended = []
        now, c = self._now(), self.counters
        for r, tok in zip(self.wanted(plan), tokens):
            if r.last_token_at is not None:
                gap = now - r.last_token_at
                c.gaps += 1
                c.gap_sum_s += gap
                c.gap_max_s = max(c.gap_max_s, gap)
            r.last_token_at = now
            r.output.append(int(tok))
            r.phase = "decode"
            length = self.cache.length(r.rid)
            if int(tok) in r.stop_ids:
                reason = "stop"
            elif len(r.output) >= r.max_new_tokens:
                reason = "length"
            elif length + 1 > self.max_context:
                reason = "context_limit"
            else:
                continue
            self._finish(r, reason)
            ended.append(r)
        return ended
