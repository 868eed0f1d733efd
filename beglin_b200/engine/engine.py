"""The engine: a model on one GPU with its cache, its step function, and generation on top.

`Engine.from_folder` reads a model folder (config.json chooses the architecture through the
registry; the tensors are bound by name).  `Engine.step` is the one step function: it runs exactly
the tokens it is given, as one batch, from and into the cache, and returns the logits at the wanted
places.  `Engine.generate` drives the scheduler and the sampler over it, host token ids in and out,
the way the reference's `greedy` mode (qwen_infer.c:20412-20429) and `cbatch` mode (:20748-20866)
drive its step functions.
"""
from __future__ import annotations

import os
from typing import Dict, Hashable, Iterable, List, Optional, Sequence, Union

import torch

from ..cache.manager import CacheManager
from ..config import load_config
from ..csrc import ops
from ..parts.context import BuildContext
from ..sampling.sampler import Sampler, uniform
from ..weights import Checkpoint, TensorDict, bind, random_tensors
from .batch import Entry, StepBatch
from .model import DecoderModel
from .portion_graph import PortionGraphs
from .scheduler import Request, Scheduler

_DTYPES = {"float32": torch.float32, "fp32": torch.float32, "f32": torch.float32,
           "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}


def parse_dtype(name: Union[str, torch.dtype]) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.float32, torch.bfloat16):
            raise ValueError(f"dtype must be float32 or bfloat16, got {name}")
        return name
    try:
        return _DTYPES[name.lower()]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got '{name}'") from None


def require_gpu(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError("beglin_b200 runs on an NVIDIA GPU (sm_100a) only: no CUDA device is available "
                           f"for '{device}', and there is no CPU path")
    ops.lib()          # builds and loads the kernels, or raises
    return device


class Engine:
    def __init__(self, spec, tensors, *, dtype="bfloat16", device="cuda:0", max_tokens: int = 8192,
                 page_size: int = 64, max_requests: int = 8, max_context: Optional[int] = None,
                 kv_split: int = 256, gemm: str = "auto", attention: str = "auto", fuse: bool = True,
                 use_graphs: bool = True, portion_graph_rows: int = 256, config=None, origin: str = ""):
        """`tensors` is anything with names()/shape(name)/tensor(name): a Checkpoint or a TensorDict.
        `max_tokens` sizes the page pool: it holds that many positions (rounded up to whole pages).
        With `use_graphs`, decoding steps and portions of one request of at least `portion_graph_rows`
        tokens whose shape comes again are replayed as CUDA graphs."""
        self.device = require_gpu(device)
        self.dtype = parse_dtype(dtype)
        self.spec, self.config = spec, config
        bound = bind(spec, tensors, origin)
        self.ctx = BuildContext(device=self.device, compute_dtype=self.dtype, page_size=page_size,
                                kv_split=kv_split, gemm=gemm, attention=attention, fuse=fuse)
        with torch.cuda.device(self.device):
            self.model = DecoderModel(spec, bound, self.ctx)
            del bound
            num_pages = max(1, -(-max_tokens // page_size))
            limit = max_context if max_context is not None else num_pages * page_size
            if spec.max_positions:
                limit = min(limit, spec.max_positions)
            self.cache = CacheManager(self.model.cache_needs(), page_size, num_pages, max_requests, limit)
            self.cache.allocate(self.device, self.dtype)
        self.sampler = Sampler(self.device)
        self.vocab = spec.vocab
        self.use_graphs = use_graphs
        self._graphs = {}
        self.portions = PortionGraphs(self, min_rows=portion_graph_rows)

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_folder(cls, folder: str, config_path: Optional[str] = None, **kw) -> "Engine":
        """`config_path` names a config.json that stands elsewhere than in the folder (the reference's
        QWEN_HF_CONFIG, qwen_infer.c:20121)."""
        ckpt = Checkpoint(folder)
        try:
            arch, cfg = load_config(config_path or folder, tensor_names=ckpt.names())
            return cls(arch.build_spec(cfg), ckpt, config=cfg, origin=folder, **kw)
        finally:
            ckpt.close()

    @classmethod
    def random(cls, config_json: dict, seed: int = 0, *, std: float = 0.02, bias_std: Optional[float] = None,
               norm_std: float = 0.02, **kw) -> "Engine":
        """Random weights made on the device, for sizes too large to write to disk first: the values of
        `write_random_model(..., generator="counter")` with the same seed, bit for bit."""
        arch, cfg = load_config(dict(config_json))
        spec = arch.build_spec(cfg)
        dtype = parse_dtype(kw.get("dtype", "bfloat16"))
        device = require_gpu(kw.get("device", "cuda:0"))
        tensors = random_tensors(spec, seed, std, bias_std, norm_std, dtype=dtype, device=str(device), generator="counter")
        return cls(spec, TensorDict(tensors), config=cfg, origin="random weights", **kw)

    # ------------------------------------------------------------------ the step function
    def step(self, entries: Sequence[Union[Entry, tuple, dict]], end: Iterable[Hashable] = (),
             check: bool = True) -> Optional[torch.Tensor]:
        """Run one batch: for every entry (request, next tokens, wanted places) exactly its tokens,
        at the positions that follow what the request already holds.  A request seen for the first
        time starts empty.  Returns float logits [wanted places, vocab] on the device, in the order
        of the entries and of their `want`, or None if nothing is wanted.  Requests named in `end`
        give back what they hold after the step."""
        ents = [self._entry(e) for e in entries]
        seen = set()
        for e in ents:
            if e.rid in seen:
                raise ValueError(f"request {e.rid!r} appears twice in one step")
            seen.add(e.rid)
            if len(e.tokens) == 0:
                raise ValueError(f"request {e.rid!r} brings no tokens")
            ids = e.ids()
            if ids.min() < 0 or ids.max() >= self.vocab:
                bad = int(ids[(ids < 0) | (ids >= self.vocab)][0])
                raise ValueError(f"request {e.rid!r}: token id {bad} is outside the vocabulary [0, {self.vocab})")
            for w in e.want:
                if not 0 <= int(w) < len(e.tokens):
                    raise ValueError(f"request {e.rid!r}: wanted place {w} is outside its {len(e.tokens)} tokens")
        logits = None
        if ents:
            new = [e.rid for e in ents if not self.cache.has(e.rid)]
            try:
                for rid in new:
                    self.cache.add_request(rid)
                plan = [(e.rid, self.cache.length(e.rid) + len(e.tokens)) for e in ents]
                self.cache.reserve(plan)
            except Exception:
                for rid in new:
                    if self.cache.has(rid):
                        self.cache.release(rid)
                raise
            try:
                logits = self.run(ents, plan)
            except Exception:
                # the step did not happen: what was reserved for it goes back, and a request that came with
                # this step is gone again
                for rid in new:
                    self.cache.release(rid)
                self.cache.trim([e.rid for e in ents])
                raise
            if check:
                ops.raise_on_status(self.ctx.status)
        for rid in end:
            if self.cache.has(rid):
                self.cache.release(rid)
        return logits

    def run(self, ents: Sequence[Entry], plan) -> Optional[torch.Tensor]:
        """The step proper, for entries whose pages are reserved: build the batch, run the model,
        record the new lengths."""
        with torch.cuda.device(self.device):
            starts = [self.cache.length(e.rid) for e in ents]
            key = self.portions.key_of(ents, starts) if self.use_graphs else None
            graph = self.portions.get(key) if key is not None else None
            if graph is not None:              # a portion of one request in a shape that came before
                logits = self.portions.step(graph, ents[0], starts[0])
            else:
                batch = StepBatch(ents, starts, self.device, self.cache)
                logits = self.model.forward(batch, self.cache)
        self.cache.commit(plan)
        return logits

    @staticmethod
    def _entry(e) -> Entry:
        if isinstance(e, Entry):
            return e
        if isinstance(e, dict):
            return Entry(e["id"], list(e["tokens"]), list(e.get("want", ())))
        rid, tokens, *rest = e
        return Entry(rid, list(tokens), list(rest[0]) if rest else [])

    def release(self, rid: Hashable) -> None:
        self.cache.release(rid)

    # ------------------------------------------------------------------ decoding as a CUDA graph
    def decode_graph(self, n: int):
        """The graph that serves decoding steps of n requests: one per bucket of batch sizes (1, 2, 4, ...),
        so requests that end one by one go through a handful of graphs, not one per count."""
        from .decode_graph import DecodeGraph, bucket
        size = bucket(n)
        g = self._graphs.get(size)
        if g is None:
            with torch.cuda.device(self.device):
                g = self._graphs[size] = DecodeGraph(self, size)
        return g

    def decode(self, rids: Sequence[Hashable], tokens: Optional[Sequence[int]] = None,
               temperatures: Optional[Sequence[float]] = None, uniforms: Optional[Sequence[float]] = None,
               read_back: bool = True):
        """One decoding step for live requests, one token each, run as a replayed CUDA graph:
        `tokens` (host ids; None feeds what the last step sampled, kept on the device) in, the
        sampled tokens out (greedy unless temperatures and uniform numbers are given)."""
        g = self.decode_graph(len(rids))
        if not g.prepared(rids):               # else the last step made room while the device was busy
            self.cache.reserve([(r, self.cache.length(r) + 1) for r in rids])
        with torch.cuda.device(self.device):
            return g.step(rids, tokens, temperatures, uniforms, read_back)

    # ------------------------------------------------------------------ generation
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: Union[int, Sequence[int]] = 32,
                 temperature: float = 0.0, seed: int = 0, stop_ids: Optional[Sequence[int]] = None,
                 max_batch: Optional[int] = None, max_step_tokens: int = 2048,
                 prefill_budget: Optional[int] = None, return_requests: bool = False, mixed: bool = True):
        """Generate for every prompt (lists of token ids on the host) and return the new token ids
        per prompt (the stop token included, as the reference records it, qwen_infer.c:2032-2039).
        `stop_ids` defaults to the configuration's eos ids; pass () to run to the token limit, as
        the reference's `greedy` mode does.  `mixed` False runs every prompt in steps of its own while the
        decoding requests wait (the reference's QWEN_CB_MIXED=0); the tokens are the same."""
        if stop_ids is None:
            stop_ids = tuple(self.spec.eos_ids)
        if isinstance(max_new_tokens, int):
            max_new_tokens = [max_new_tokens] * len(prompts)
        sched = Scheduler(self.cache, max_batch=max_batch or self.cache.max_requests,
                          max_step_tokens=max_step_tokens, prefill_budget=prefill_budget, mixed=mixed)
        reqs = []
        for i, (p, n) in enumerate(zip(prompts, max_new_tokens)):
            bad = [t for t in p if not 0 <= int(t) < self.vocab]
            if bad:
                raise ValueError(f"prompt {i}: token id {bad[0]} is outside the vocabulary [0, {self.vocab})")
            r = Request(rid=("gen", i), prompt=[int(t) for t in p], max_new_tokens=int(n),
                        temperature=float(temperature), seed=int(seed), stop_ids=tuple(stop_ids))
            reqs.append(r)
            if n <= 0:
                r.phase, r.finish_reason = "done", "length"
            else:
                sched.add(r)
        try:
            while True:
                plan = sched.plan()
                if plan is None:
                    break
                wanted = sched.wanted(plan)
                temps = [r.temperature for r in wanted]
                us = [uniform(r.seed, r.rid[1], len(r.output)) if r.temperature > 0 else 0.0 for r in wanted]
                tokens: List[int] = []
                if self.use_graphs and not plan.prefill:
                    with torch.cuda.device(self.device):
                        tokens = self.decode_graph(len(wanted)).step(
                            [r.rid for r in wanted], [r.output[-1] for r in wanted], temps, us)
                else:
                    logits = self.run(plan.entries, plan.lengths)
                    if wanted:
                        tokens = self.sampler.sample(logits, temps, us)
                sched.update(plan, tokens, committed=True)      # the step functions above have recorded the lengths
            ops.raise_on_status(self.ctx.status)
        finally:
            for r in list(sched.running):
                if self.cache.has(r.rid):
                    self.cache.release(r.rid)
        self.last_counters = sched.counters
        if return_requests:
            return reqs
        return [list(r.output) for r in reqs]
