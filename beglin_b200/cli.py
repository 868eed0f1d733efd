"""The command line in the reference's manner: `qwen_infer <mode> <N>` with everything else in
environment variables (qwen_infer.c:20108-20128).

Modes kept: `greedy` (default; N new tokens, default 32, no stop on EOS, output `greedy: id id ...`,
qwen_infer.c:20412-20429), `ppl` (teacher-forced perplexity over the first N, default 12, token files
<QWEN_BASE>/eval/ppl_work/w0.i32, w1.i32, ..., output `ppl P tokens T`, :20488-20504), `bench` (prefill,
8 warm-up tokens, N timed decode tokens, best of 3, output `tok_s ... ms_tok ...`, :20430-20462), `dump`
(last logits of the prompt to a file,
:20405-20411) and `cbatch` (continuous batching over prompts cut from the loaded one, output one
`cbatch req...` line per request and an `agg_tok_s` line with the reference's `util`, `avg_active`,
`steps`, `msteps`, `pfonly`, `pf_cols`, `tbt_max_ms` and `tbt_mean_ms` fields, :20611-20912).

Variables kept, with the reference's meanings: QWEN_BASE (here: the model folder with config.json
and model.safetensors), QWEN_PROMPT (file of little-endian int32 token ids; default
<QWEN_BASE>/ref/prompt_ids.i32), QWEN_SAFETENSORS_MAXSEQ (context cap, default 2048), QWEN_BATCH
(live requests, default 8), QWEN_CB_REQS (default 12), QWEN_CB_REPS (default 3),
QWEN_CB_PREFILL_BUDGET (prompt tokens per step, default 16), QWEN_CB_STOP_EXTRA (an extra stop id),
QWEN_CB_MIXED (default 1; 0 runs every prompt in steps of its own while the decoding requests wait, for the
comparison of the two orders, qwen_infer.c:20690), QWEN_HF_CONFIG (a config.json that stands elsewhere than in
the model folder, :20121), QWEN_PROF (1: in `bench` and `greedy`, device time per kernel class from CUDA events,
printed with the share of the total that the classes add up to, :1224-1235 and :20463-20486; the steps then
run kernel by kernel, not as replayed graphs).
Added: QWEN_DTYPE (bf16 | fp32, default bf16), QWEN_TEMPERATURE and QWEN_SEED (sampling),
QWEN_PAGE_SIZE (default 64), QWEN_NUM_PAGES, QWEN_RANDOM (a seed: write random weights for
<QWEN_BASE>/config.json first, if the folder has no model.safetensors), QWEN_DUMP_DIR.
"""
from __future__ import annotations

import os
import sys
import time
from typing import List

import numpy as np


def _env_int(name: str, default: int) -> int:
    v = os.environ.get(name)
    return int(v) if v else default


def _err(msg: str) -> int:
    print(f"FATAL: {msg}", file=sys.stderr)
    return 1


def load_ids(path: str, limit: int) -> List[int]:
    """Raw little-endian int32 ids (qwen_infer.c:2168-2170)."""
    return np.fromfile(path, dtype="<i4")[:limit].astype(np.int64).tolist()


class PhaseReport:
    """QWEN_PROF: device time per kernel class between its making and `close`, measured with CUDA events
    around every launch of the class, against the device time of the whole stretch.  The classes do not add
    up to the total: what is missing is the time in which no kernel of the package ran (launch gaps of steps
    that run kernel by kernel, library products of steps of many rows).  The closing line says how much they
    cover, as the reference's does (qwen_infer.c:20463-20467)."""

    def __init__(self, ops):
        import torch
        self.ops, self.torch = ops, torch
        self.t0, self.t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ops.profile_begin()
        self.t0.record()
        self.phases = None

    def close(self) -> None:
        if self.phases is None:
            self.t1.record()
            self.phases = self.ops.profile_end()
            self.total_ms = self.t0.elapsed_time(self.t1)

    def print(self, ctx: int, n: int, unit: str) -> None:
        self.close()
        total = self.total_ms / n
        covered = sum(ms for ms, _ in self.phases.values()) / n
        print(f"[prof] ctx~{ctx} total={total:.3f}ms/{unit} sum(phases)={covered:.3f}ms/{unit} "
              f"closure={100.0 * covered / total if total > 0 else 0.0:.1f}%", file=sys.stderr)
        for name, (ms, count) in self.phases.items():
            print(f"[prof]   {name:14s} {ms / n:.4f} ms ({100.0 * ms / n / total if total > 0 else 0.0:.2f}%) in {count} brackets",
                  file=sys.stderr)
        print(f"PROF ctx {ctx} total_ms {total:.4f} " + " ".join(f"{k} {ms / n:.4f}" for k, (ms, _) in self.phases.items()))


def describe(spec) -> str:
    """The reference's arch line (qwen_infer.c:19489-19490) from a model's description: the sizes are read
    off the parts of the first layer, whatever architecture built the description; a size that the layer's
    parts do not have is left out."""
    first = spec.layers[0].parts if spec.layers else {}
    mixer, ff = first.get("mixer"), first.get("feed_forward")
    fields = [("NL", len(spec.layers)), ("NH", getattr(mixer, "n_heads", None)), ("NKV", getattr(mixer, "n_kv_heads", None)),
              ("D", spec.hidden), ("HD", getattr(mixer, "head_dim", None)), ("IM", getattr(ff, "intermediate", None)),
              ("VOCAB", spec.vocab)]
    position = getattr(mixer, "position", None)
    theta = getattr(position, "theta", None)
    if theta is not None:
        fields.append(("THETA", f"{theta:.1f}"))
    fields.append(("EPS", f"{spec.final_norm.eps:g}"))
    if getattr(mixer, "qkv_bias", None) is not None:
        fields.append(("QKV_BIAS", int(mixer.qkv_bias)))
    if getattr(mixer, "n_heads", None) and getattr(mixer, "n_kv_heads", None):
        fields.append(("GROUP", mixer.n_heads // mixer.n_kv_heads))
    return " ".join(f"{k}={v}" for k, v in fields if v is not None)


def main(argv: List[str]) -> int:
    mode = argv[1] if len(argv) > 1 else "greedy"
    n_gen = int(argv[2]) if len(argv) > 2 else 32
    if mode in ("-h", "--help"):
        print(__doc__)
        return 0
    if mode not in ("greedy", "bench", "dump", "ppl", "cbatch"):
        return _err(f"unknown mode '{mode}'; modes: greedy, bench, dump, ppl, cbatch")
    base = os.environ.get("QWEN_BASE")
    if not base:
        return _err("QWEN_BASE is not set (the model folder with config.json and model.safetensors)")
    config_path = os.environ.get("QWEN_HF_CONFIG") or os.path.join(base, "config.json")
    if not os.path.exists(config_path):
        return _err(f"{config_path}: no arch config (config.json) found")
    prof = bool(_env_int("QWEN_PROF", 0))

    import torch
    from .engine.engine import Engine
    from .csrc import ops

    maxseq = _env_int("QWEN_SAFETENSORS_MAXSEQ", 2048)
    dtype = os.environ.get("QWEN_DTYPE", "bf16")
    page = _env_int("QWEN_PAGE_SIZE", 64)
    batch = max(1, _env_int("QWEN_BATCH", 8))
    seed_random = os.environ.get("QWEN_RANDOM")
    if seed_random and not os.path.exists(os.path.join(base, "model.safetensors")) \
            and not os.path.exists(os.path.join(base, "model.safetensors.index.json")):
        import json
        from .weights import write_random_model
        with open(config_path) as f:
            cfg_json = json.load(f)
        print(f"[engine] writing random weights (seed {seed_random}) to {base}", file=sys.stderr)
        write_random_model(base, cfg_json, int(seed_random),
                           dtype=torch.float32 if dtype in ("fp32", "float32") else torch.bfloat16)

    prompt_path = os.environ.get("QWEN_PROMPT") or os.path.join(base, "ref", "prompt_ids.i32")
    prompt: List[int] = []
    if mode != "ppl":                                        # ppl reads its own token files (qwen_infer.c:20402)
        try:
            prompt = load_ids(prompt_path, maxseq)
        except OSError as e:
            return _err(f"could not read prompt ids from {prompt_path} ({e.strerror})")
        if len(prompt) < 1:
            return _err(f"no prompt ids (np={len(prompt)})")

    live = batch if mode == "cbatch" else 1
    num_pages = _env_int("QWEN_NUM_PAGES", live * -(-maxseq // page))
    try:
        eng = Engine.from_folder(base, config_path=config_path, dtype=dtype, max_tokens=num_pages * page, page_size=page,
                                 max_requests=live, max_context=maxseq, use_graphs=not prof)
    except Exception as e:                                   # one line, as the reference's FATALs
        return _err(str(e))
    print(f"[engine] arch config ({config_path}): {describe(eng.spec)} MAXSEQ={maxseq} DTYPE={dtype}", file=sys.stderr)
    temperature = float(os.environ.get("QWEN_TEMPERATURE", "0"))
    seed = _env_int("QWEN_SEED", 0)

    if mode == "dump":
        logits = eng.step([("dump", prompt, [len(prompt) - 1])], end=["dump"])
        out_dir = os.environ.get("QWEN_DUMP_DIR") or os.path.join(base, "results")
        os.makedirs(out_dir, exist_ok=True)
        logits[0].cpu().numpy().astype("<f4").tofile(os.path.join(out_dir, "c_logits_last.f32"))
        print(f"[engine] dumped, argmax={int(eng.sampler.greedy(logits)[0])}", file=sys.stderr)
        return 0

    if mode == "ppl":
        n_win = int(argv[2]) if len(argv) > 2 else 12
        tot_nll, tot, rows = 0.0, 0, 256                     # the logits of 256 places at a time
        for wi in range(n_win):
            try:
                ids = load_ids(os.path.join(base, "eval", "ppl_work", f"w{wi}.i32"), maxseq)
            except OSError:
                continue
            if len(ids) < 2:
                continue
            for lo in range(0, len(ids), rows):
                part = ids[lo:lo + rows]
                want = [i for i in range(len(part)) if lo + i < len(ids) - 1]      # every place but the window's last
                logits = eng.step([("ppl", part, want)], end=["ppl"] if lo + rows >= len(ids) else [])
                if want:
                    nxt = torch.tensor(ids[lo + 1:lo + 1 + len(want)], device=logits.device)
                    lg = logits.double()
                    nll = torch.logsumexp(lg, dim=1) - lg.gather(1, nxt[:, None])[:, 0]
                    tot_nll += float(nll.sum())
                    tot += len(want)
            print(f"[ppl] window {wi} done ({tot} toks)", file=sys.stderr)
        if tot == 0:
            return _err("no ppl tokens (missing eval/ppl_work?)")
        import math
        ppl = math.exp(tot_nll / tot)
        print(f"[ppl] {dtype} ppl {ppl:.4f} over {tot} tokens", file=sys.stderr)
        print(f"ppl {ppl:.4f} tokens {tot}")
        return 0

    if mode == "greedy":
        room = maxseq - len(prompt)
        n_new = min(n_gen, max(room, 0) + 1)
        timer = PhaseReport(ops) if prof else None
        out = eng.generate([prompt], max_new_tokens=n_new, temperature=temperature, seed=seed, stop_ids=())[0]
        if timer:
            timer.print(len(prompt) + len(out), max(1, len(prompt) + len(out) - 1), "tok (prompt and new)")
        print("greedy:" + "".join(f" {t}" for t in out))
        return 0

    if mode == "bench":
        N = n_gen
        if len(prompt) + 8 + N >= maxseq:
            old, N = N, maxseq - len(prompt) - 8 - 1
            if N < 1:
                return _err(f"prompt too long for bench (np={len(prompt)})")
            print(f"[bench] N clamped {old}->{N} to fit MAXSEQ={maxseq}", file=sys.stderr)
        best = float("inf")
        for _ in range(3):
            logits = eng.step([("b", prompt, [len(prompt) - 1])])
            tok = eng.sampler.greedy(logits)
            for _ in range(8):
                logits = eng.step([("b", [int(tok[0])], [0])])
                tok = eng.sampler.greedy(logits)
            torch.cuda.synchronize()
            timer = PhaseReport(ops) if prof else None
            t0 = time.perf_counter()
            for _ in range(N):
                logits = eng.step([("b", [int(tok[0])], [0])], check=False)
                tok = eng.sampler.greedy(logits)
            torch.cuda.synchronize()
            took = time.perf_counter() - t0
            if timer:
                timer.close()
                if took < best:
                    best_timer = timer
            best = min(best, took)
            eng.release("b")
        if prof:
            best_timer.print(len(prompt) + 8, N, "tok")
        ms = best / N * 1e3
        print(f"[bench] {dtype} N={N} pos~{len(prompt) + 8}: {ms:.3f} ms/tok = {1000.0 / ms:.2f} tok/s", file=sys.stderr)
        print(f"tok_s {1000.0 / ms:.3f} ms_tok {ms:.2f}")
        return 0

    # cbatch: prompts cut from the loaded one, lengths 4..40 and token limits spread as in the reference
    R = max(1, _env_int("QWEN_CB_REQS", 12))
    reps = max(1, _env_int("QWEN_CB_REPS", 3))
    budget = max(1, _env_int("QWEN_CB_PREFILL_BUDGET", 16))
    stop_extra = _env_int("QWEN_CB_STOP_EXTRA", -1)
    mixed = bool(_env_int("QWEN_CB_MIXED", 1))
    spread = n_gen if n_gen > 1 else 27
    plen = [min(len(prompt), 4 + (r * 13) % 37) for r in range(R)]
    maxnew = [6 + (r * 7) % spread for r in range(R)]
    stops = tuple(eng.spec.eos_ids) + ((stop_extra,) if stop_extra >= 0 else ())
    best_wall, first, identical, reqs, c = float("inf"), None, True, None, None
    for _ in range(reps):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        reqs = eng.generate([prompt[:n] for n in plen], max_new_tokens=maxnew, temperature=temperature, seed=seed,
                            stop_ids=stops, max_batch=batch, prefill_budget=budget, return_requests=True, mixed=mixed)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        if wall < best_wall:
            best_wall, c = wall, eng.last_counters          # the counters of the fastest repeat, as the reference keeps
        outs = [r.output for r in reqs]
        if first is None:
            first = outs
        elif outs != first:
            identical = False
    tot = sum(len(r.output) for r in reqs)
    for i, r in enumerate(reqs):
        print(f"cbatch req{i} plen {plen[i]} maxnew {maxnew[i]} nout {len(r.output)}:" + "".join(f" {t}" for t in r.output))
    print(f"agg_tok_s {tot / best_wall:.3f} wall_s {best_wall:.3f} util {c.utilisation(batch):.4f} "
          f"avg_active {c.decode_rows / max(1, c.steps):.3f} B {batch} R {R} tok {tot} reps_identical "
          f"{int(identical)} mixed {int(mixed)} steps {c.steps} msteps {c.mixed_steps} pfonly {c.prefill_only_steps} "
          f"pstall {c.prefill_stalls} pf_cols {c.prefill_rows} tbt_max_ms {c.gap_max_s * 1e3:.3f} tbt_mean_ms {c.gap_mean_s() * 1e3:.3f} "
          f"preemptions {c.preemptions}")
    return 0
