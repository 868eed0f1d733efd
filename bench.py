#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen2.5-1.5B layer sizes, random weights, bf16.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 4096] [--layers N] [--sizes 1.5b]
    python bench.py --impl reference ...      # prints the reference arm's `unavailable` line

A step is one decoding step of `batch` requests, each holding close to `context` positions in the
paged cache.  It prints ONE JSON line: `value` is decoded tokens a second on the device (the step
replayed as a CUDA graph, sampled tokens fed back on the device); `e2e` is the same through the
Python entry point `Engine.decode`, host token ids in from pinned memory and sampled ids read back
every step; `prefill` is one 2,048-token prompt in one step; `roofline` sets the bytes a decoding
step has to read (every weight once and the cache of the live requests) against the measured copy
bandwidth; `points` holds decoding at batch 1 and 64, and the other configurations of the baseline
record, each with its own engine, built and freed in turn: `decode_b8_page16` (the headline sizes with
pages of 16 positions), `gen_7b_*` (Qwen2.5-7B sizes, context 8192: 32 requests with seeded prompt lengths
of 128 to 2,048 tokens and 256 new tokens each through `Engine.generate`) and `decode_14b_b64` (Qwen2.5-14B
sizes, 64 prompts of 4,096 tokens, context limit 16384), the decoding points with milliseconds per step and
their fraction of the copy bandwidth.  `--no-big` leaves the 7B and 14B points out.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Qwen2.5-1.5B layer sizes: the third configuration of the baseline record.
CONFIG_1P5B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 28, "hidden_size": 1536, "num_attention_heads": 12, "num_key_value_heads": 2,
    "intermediate_size": 8960, "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "use_sliding_window": False, "hidden_act": "silu",
    "max_position_embeddings": 32768,
}
# Other layer sizes of the same architecture, for measurements beside the default one (--sizes).
_BIG = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "rope_theta": 1000000.0, "use_sliding_window": False,
        "hidden_act": "silu", "max_position_embeddings": 32768, "tie_word_embeddings": False, "vocab_size": 152064}
SIZES = {
    "1.5b": ("Qwen2.5-1.5B", CONFIG_1P5B),
    "0.5b": ("Qwen2.5-0.5B", dict(CONFIG_1P5B, num_hidden_layers=24, hidden_size=896, num_attention_heads=14,
                                  intermediate_size=4864)),
    "7b": ("Qwen2.5-7B", dict(_BIG, num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4,
                              intermediate_size=18944, rms_norm_eps=1e-6)),
    "14b": ("Qwen2.5-14B", dict(_BIG, num_hidden_layers=48, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
                                intermediate_size=13824, rms_norm_eps=1e-5)),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        out = {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
        if "bf16_tflops_sustained" in p:
            out["bf16_tflops_sustained"] = float(p["bf16_tflops_sustained"])
        return out
    except (OSError, KeyError, ValueError, TypeError):
        return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.samples, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm = sorted(int(s[0]) for s in self.samples if s[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower() == "active" for s in self.samples)]
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}


def kv_bytes_per_token(cfg, layers):
    hd = cfg["hidden_size"] // cfg["num_attention_heads"]
    return layers * 2 * cfg["num_key_value_heads"] * hd * 2


def prefill_flops(cfg, layers, T):
    d, im, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    hd = d // cfg["num_attention_heads"]
    qd, kvd = cfg["num_attention_heads"] * hd, cfg["num_key_value_heads"] * hd
    linear = 2.0 * T * layers * (d * (qd + 2 * kvd) + qd * d + 3 * d * im)
    attn = layers * 4.0 * qd * (T * (T + 1) / 2.0)
    head = 2.0 * d * V                     # the last row only
    return linear + attn + head


def fill_cache(eng, rids, length, seed, chunk=2048):
    """Prefill every request to `length` positions with seeded uniform token ids, through the step
    function, a few requests at a time."""
    import torch
    g = torch.Generator().manual_seed(seed)
    per_step = max(1, 8192 // min(length, chunk))
    for lo in range(0, len(rids), per_step):
        group = rids[lo:lo + per_step]
        ids = {r: torch.randint(0, eng.vocab, (length,), generator=g).tolist() for r in group}
        for p in range(0, length, chunk):
            eng.step([(r, ids[r][p:p + chunk], []) for r in group], check=False)
    torch.cuda.synchronize()


def time_decode(eng, batch, context, steps, warmup, seed, e2e, start_len=None):
    """(ms per step on the device, launches of this package's kernels in the timed region).  With
    `e2e` every step takes its tokens from the host and reads the sampled ones back.  The requests hold
    `start_len` positions before the first step (default: so that the last timed step ends at `context`)."""
    import torch
    from beglin_b200.csrc import ops
    rids = [("bench", batch, i) for i in range(batch)]
    if start_len is None:
        start_len = context - (warmup + steps) - 1
    fill_cache(eng, rids, start_len, seed)
    g = torch.Generator().manual_seed(seed + 1)
    toks = torch.randint(0, eng.vocab, (batch,), generator=g).tolist()
    if e2e:
        for _ in range(warmup):
            toks = eng.decode(rids, toks, read_back=True)
    else:
        eng.decode(rids, toks, read_back=False)          # host tokens once; then fed back on the device
        for _ in range(warmup - 1):
            eng.decode(rids, None, read_back=False)
    torch.cuda.synchronize()
    before = ops.launch_count()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    h2d = 0
    if e2e:
        for _ in range(steps):
            toks = eng.decode(rids, toks, read_back=True)
            h2d += eng.decode_graph(batch).h2d_bytes
    else:
        for _ in range(steps):
            eng.decode(rids, None, read_back=False)
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1) / steps
    launches = ops.launch_count() - before
    ops.raise_on_status(eng.ctx.status)
    for r in rids:
        eng.release(r)
    return ms, launches, h2d / steps


def decode_timeline(eng, batch, context, seed):
    """The kernels of ONE decode step as the device ran them (CUPTI records through torch.profiler): for
    every kernel its start and end relative to the step's first kernel, in microseconds.  Under
    programmatic dependent launch a kernel starts while the one before it still runs and then waits, so
    what a kernel adds to the step is the difference between its end and the end of the kernel before."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    rids = [("timeline", batch, i) for i in range(batch)]
    fill_cache(eng, rids, context - 16, seed)
    toks = torch.randint(0, eng.vocab, (batch,), generator=torch.Generator().manual_seed(seed)).tolist()
    eng.decode(rids, toks, read_back=False)
    for _ in range(4):
        eng.decode(rids, None, read_back=False)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(2):
            eng.decode(rids, None, read_back=False)
        torch.cuda.synchronize()
    ev = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA
          and "memcpy" not in e.name.lower() and "memset" not in e.name.lower()]
    ev.sort(key=lambda e: e.time_range.start)
    first = [i for i, e in enumerate(ev) if "embed_gather" in e.name][-1]
    step = ev[first:]
    t0 = step[0].time_range.start
    for r in rids:
        eng.release(r)

    def short(name):
        return name.replace("void bg::", "").replace("bg::", "").split("<")[0].split("(")[0]
    return [(short(e.name), e.time_range.start - t0, e.time_range.end - t0) for e in step]


def print_timeline(rows, layers):
    print(f"{len(rows)} kernels, {rows[-1][2]:.1f} us from the first kernel's start to the last one's end")
    print("  #  kernel                               start      end   adds")
    prev = 0.0
    shown = list(range(min(len(rows), 24))) + list(range(max(24, len(rows) - 6), len(rows)))
    for i, (name, s, e) in enumerate(rows):
        if i in shown:
            print(f"{i:4d} {name[:34]:34s} {s:8.1f} {e:8.1f} {e - prev:6.1f}")
        elif i == 24:
            print("     ...")
        prev = max(prev, e)
    adds, prev = {}, 0.0
    for name, s, e in rows:
        a = adds.setdefault(name, [0, 0.0])
        a[0] += 1
        a[1] += max(0.0, e - prev)
        prev = max(prev, e)
    print("what each kind of kernel adds to the step (its end minus the end of the kernel before it):")
    for name, (n, t) in sorted(adds.items(), key=lambda kv: -kv[1][1]):
        print(f"  {name[:40]:40s} x{n:<4d} {t:8.1f} us  ({t / n:5.1f} us each)")


def prefill_timeline(eng, T, seed):
    """The kernels of ONE prompt step of T tokens as the device ran them: (name, start, end) in microseconds
    from the step's first kernel, library kernels included."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, eng.vocab, (T,), generator=g).tolist()
    for _ in range(3):
        eng.step([("timeline", ids, [T - 1])], end=["timeline"], check=False)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        eng.step([("timeline", ids, [T - 1])], end=["timeline"], check=False)
        torch.cuda.synchronize()
    ev = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA
          and "memcpy" not in e.name.lower() and "memset" not in e.name.lower()]
    ev.sort(key=lambda e: e.time_range.start)
    t0 = ev[0].time_range.start

    def short(name):
        return name.replace("void bg::", "").replace("bg::", "").split("<")[0].split("(")[0]
    return [(short(e.name), e.time_range.start - t0, e.time_range.end - t0) for e in ev]


def print_busy(rows):
    """Per kind of kernel the time it ran (not what it adds), and the time in which the device ran nothing."""
    busy, idle, prev = {}, 0.0, 0.0
    for name, s, e in rows:
        b = busy.setdefault(name, [0, 0.0])
        b[0] += 1
        b[1] += e - s
        idle += max(0.0, s - prev)
        prev = max(prev, e)
    print(f"the device ran nothing for {idle:.1f} us of the step; time each kind of kernel ran:")
    for name, (n, t) in sorted(busy.items(), key=lambda kv: -kv[1][1]):
        print(f"  {name[:40]:40s} x{n:<4d} {t:8.1f} us  ({t / n:6.1f} us each)")


def time_prefill(eng, T, reps, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    best = float("inf")
    for i in range(reps + 2):
        ids = torch.randint(0, eng.vocab, (T,), generator=g).tolist()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        eng.step([("prefill", ids, [T - 1])], end=["prefill"], check=False)
        t1.record()
        torch.cuda.synchronize()
        if i >= 2:
            best = min(best, t0.elapsed_time(t1))
    return best


def free_engine(eng):
    """Drop an engine and everything it holds on the device (its graphs refer back to it, so the cycle
    collector has to run before the memory is free)."""
    import gc
    import torch
    eng._graphs.clear()
    eng.portions.graphs.clear()
    del eng
    gc.collect()
    torch.cuda.empty_cache()


def decode_point(cfg, pk, batch, context, start_len, steps, warmup, page, max_context=None, seed=5):
    """One decoding measurement with an engine of its own: tokens a second, milliseconds a step, the bytes a
    step has to read and their fraction of the copy bandwidth."""
    from beglin_b200 import Engine
    layers = cfg["num_hidden_layers"]
    eng = Engine.random(cfg, seed=0, dtype="bfloat16", device="cuda:0", max_tokens=batch * (context + 2 * page), page_size=page,
                        max_requests=batch, max_context=max_context or context)
    weight_bytes = eng.model.weight_bytes()
    ms, _, _ = time_decode(eng, batch, context, steps, warmup, seed=seed, e2e=False, start_len=start_len)
    free_engine(eng)
    first = start_len if start_len is not None else context - (warmup + steps) - 1
    mid = first + warmup + steps / 2.0
    step_bytes = weight_bytes + batch * mid * kv_bytes_per_token(cfg, layers)
    gbs = step_bytes / (ms * 1e-3) / 1e9
    return {"tok_s": round(batch * 1000.0 / ms, 1), "ms": round(ms, 4), "gb": round(step_bytes / 1e9, 3),
            "frac": round(gbs / pk["hbm_gbs"], 4), "steps": steps}


def generate_point(cfg, requests=32, new_tokens=256, context=8192, seed=11):
    """The mixed workload of the baseline record's fourth configuration through `Engine.generate`: `requests`
    prompts of seeded lengths 128..2,048 (seeded uniform token ids), `new_tokens` new tokens each, all live at
    once, host token ids in and out.  The first run captures the graphs; the second is timed on the host's
    clock between two device synchronisations."""
    import torch
    from beglin_b200 import Engine
    g = torch.Generator().manual_seed(seed)
    lengths = torch.randint(128, 2049, (requests,), generator=g).tolist()
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lengths]
    eng = Engine.random(cfg, seed=0, dtype="bfloat16", device="cuda:0", max_tokens=requests * (2048 + new_tokens + 64),
                        page_size=64, max_requests=requests, max_context=context)
    out = {}
    for timed in (False, True):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = eng.generate(prompts, max_new_tokens=new_tokens, stop_ids=(), max_batch=requests, max_step_tokens=4096)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        c = eng.last_counters
        new = sum(len(o) for o in outs)
        out = {"new_tok_s": round(new / wall, 1), "tok_s_with_prompts": round((new + sum(lengths)) / wall, 1),
               "wall_s": round(wall, 3), "prompt_tokens": sum(lengths), "new_tokens": new, "steps": c.steps,
               "mixed_steps": c.mixed_steps, "preemptions": c.preemptions,
               "tbt_max_ms": round(c.gap_max_s * 1e3, 2), "tbt_mean_ms": round(c.gap_mean_s() * 1e3, 3)}
    free_engine(eng)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--sizes", default="1.5b", choices=sorted(SIZES), help="layer sizes (default: the baseline record's)")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (default: all)")
    ap.add_argument("--no-points", action="store_true", help="skip decoding at batch 1 and 64 and the prefill")
    ap.add_argument("--no-big", action="store_true", help="skip the points with engines of their own (page 16, 7B, 14B)")
    ap.add_argument("--gemm", default="auto")
    ap.add_argument("--no-fuse", action="store_true", help="norms, residual adds and SwiGLU as kernels of their own")
    ap.add_argument("--timeline", nargs="?", const="decode", default=None, choices=["decode", "prefill"],
                    help="instead of the measurement: print the kernels of one decode step (or of one prompt step of "
                         "2,048 tokens) with their device times")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a C program for Apple CPUs (Accelerate, NEON, SME2) with no Python "
                          "package: pip reports \"Neither 'setup.py' nor 'pyproject.toml' found\", and "
                          "qwen_infer.c does not compile on x86 Linux"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(3, args.warmup)
    if args.steps + args.warmup + 2 > args.context:          # every timed step decodes one more position
        args.context = args.steps + args.warmup + 64

    import torch
    from beglin_b200 import Engine
    pk = peaks()
    model_name, full = SIZES[args.sizes]
    args.layers = args.layers or full["num_hidden_layers"]
    cfg = dict(full, num_hidden_layers=args.layers)
    max_batch = args.batch if args.no_points else max(args.batch, 64)
    page = 64
    eng = Engine.random(cfg, seed=0, dtype="bfloat16", device="cuda:0", max_tokens=max_batch * args.context,
                        page_size=page, max_requests=max_batch, max_context=args.context, gemm=args.gemm, fuse=not args.no_fuse)
    if args.timeline == "prefill":
        rows = prefill_timeline(eng, 2048, seed=3)
        print_timeline(rows, args.layers)
        print_busy(rows)
        return 0
    if args.timeline:
        print_timeline(decode_timeline(eng, args.batch, args.context, seed=1), args.layers)
        return 0
    weight_bytes = eng.model.weight_bytes()
    kvb = kv_bytes_per_token(cfg, args.layers)

    clocks = ClockSampler()
    clocks.start()
    ms, launches, _ = time_decode(eng, args.batch, args.context, args.steps, args.warmup, seed=1, e2e=False)
    clock_rec = clocks.stop()
    ms_e2e, _, h2d = time_decode(eng, args.batch, args.context, args.steps, args.warmup, seed=1, e2e=True)

    value = args.batch * 1000.0 / ms
    ctx_mid = args.context - 1 - args.steps / 2.0
    step_bytes = weight_bytes + args.batch * ctx_mid * kvb
    achieved = step_bytes / (ms * 1e-3) / 1e9
    out = {
        "metric": f"decode tok/s @ batch {args.batch}; {model_name} bf16", "value": round(value, 1), "unit": "tok/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (seeded uniform token ids, random weights)",
        "config": {"model": f"{model_name} sizes", "layers": args.layers, "layers_of_config": full["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["hidden_size"] // cfg["num_attention_heads"], "intermediate": cfg["intermediate_size"],
                   "vocab": cfg["vocab_size"], "tied_head": bool(cfg["tie_word_embeddings"]), "global_batch": args.batch, "seq_len": args.context,
                   "page_size": page, "parallelism": "single GPU", "weights": "random, seeded",
                   "l2": "inputs larger than L2 (weights and cache read once per step)",
                   "peaks": pk["source"]},
        "e2e": {"value": round(args.batch * 1000.0 / ms_e2e, 1), "unit": "tok/s",
                "h2d_bytes_per_step": round(h2d, 1),
                "d2h_bytes_per_step": int(args.batch * 4)},
        "gpu_launches": int(launches),
        "clocks": clock_rec,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }
    if not args.no_points:
        points = {}
        for b in (1, 64):
            m, _, _ = time_decode(eng, b, args.context, min(args.steps, 32), args.warmup, seed=2, e2e=False)
            points[f"decode_b{b}"] = round(b * 1000.0 / m, 1)
        out["points"] = points
        T = 2048
        pms = time_prefill(eng, T, reps=3, seed=3)
        flops = prefill_flops(cfg, args.layers, T)
        out["prefill"] = {"value": round(T * 1000.0 / pms, 1), "tokens": T, "ms": round(pms, 3),
                          "frac": round(flops / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
        if not args.no_big and args.sizes == "1.5b" and args.layers == full["num_hidden_layers"]:
            free_engine(eng)
            del eng
            # the headline sizes with the page size the baseline record states
            p16 = decode_point(cfg, pk, args.batch, args.context, None, min(args.steps, 32), args.warmup, page=16)
            points.update({"decode_b8_page16": p16["tok_s"], "decode_b8_page16_ms": p16["ms"], "decode_b8_page16_frac": p16["frac"]})
            # Qwen2.5-7B sizes: the mixed workload through Engine.generate
            gen = generate_point(SIZES["7b"][1])
            points.update({"gen_7b_" + k: v for k, v in gen.items()})
            # Qwen2.5-14B sizes: 64 prompts of 4,096 tokens under a context limit of 16384
            big = decode_point(SIZES["14b"][1], pk, 64, 4096 + 64, 4096, 8, 3, page=64, max_context=16384)
            points.update({"decode_14b_b64": big["tok_s"], "decode_14b_b64_ms": big["ms"], "decode_14b_b64_gb": big["gb"],
                           "decode_14b_b64_frac": big["frac"], "decode_14b_b64_steps": big["steps"]})
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
