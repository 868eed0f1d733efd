"""Generation through the entry points: greedy against the plain implementation, temperature
sampling reproducible and independent of the batch, few pages (preemption and recomputation), and
the command line."""
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import TINY, TOL_BF16, TOL_F32, follows_plain, make_model, plain, plain_logits, plain_model, rel_err, seeded_ids

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def engine(folder, dtype, **kw):
    from beglin_b200 import Engine
    args = dict(dtype=dtype, max_tokens=512, page_size=8, max_requests=4)
    args.update(kw)
    return Engine.from_folder(folder, **args)


def test_greedy_float32_equals_plain(model_root):
    """Tiny A: prompts of 5 and 11 tokens, 8 greedy steps each."""
    folder = make_model(model_root, "A", seed=3, dtype=torch.float32)
    cfg, w = plain_model(folder)
    prompts = [seeded_ids(5, 256, 1), seeded_ids(11, 256, 2)]
    want = [plain.greedy_generate(cfg, w, p, 8) for p in prompts]
    eng = engine(folder, "float32")
    assert eng.generate(prompts, max_new_tokens=8, stop_ids=()) == want
    # one at a time gives the same
    assert [eng.generate([p], max_new_tokens=8, stop_ids=())[0] for p in prompts] == want
    assert not eng.cache.live() and eng.cache.free_pages() == eng.cache.num_pages


@pytest.mark.parametrize("name,std", [("B", 0.06), ("D", 0.08)])
def test_greedy_bfloat16_follows_plain_up_to_near_ties(model_root, name, std):
    """Weights wide enough that a row of logits is not flat: most tokens are then pinned to the plain argmax."""
    cfg, _, page = TINY[name]
    folder = make_model(model_root, name, seed=33, dtype=torch.bfloat16, std=std)
    prompts = [seeded_ids(9, cfg["vocab_size"], 4), seeded_ids(20, cfg["vocab_size"], 5), seeded_ids(33, cfg["vocab_size"], 6)]
    eng = engine(folder, "bfloat16", page_size=page)
    outs = eng.generate(prompts, max_new_tokens=12, stop_ids=())
    pinned = 0
    for p, out in zip(prompts, outs):
        assert len(out) == 12
        pinned += follows_plain(folder, p, out, tol=1e-2)
    assert pinned >= 18                                   # of 36 tokens


@pytest.mark.parametrize("budget", [4, 8, 16])
def test_bfloat16_steps_that_mix_decoding_rows_with_portions(model_root, budget):
    """Five prompts, three live at a time, a small token budget: most steps carry decoding rows beside a prompt
    portion, and the batch of decoding rows shrinks and grows.  Every token follows the plain implementation."""
    cfg, _, page = TINY["D"]
    folder = make_model(model_root, "D", seed=33, dtype=torch.bfloat16, std=0.08)
    prompts = [seeded_ids(n, cfg["vocab_size"], 60 + n) for n in (23, 7, 41, 15, 30)]
    eng = engine(folder, "bfloat16", page_size=page, max_requests=3)
    outs = eng.generate(prompts, max_new_tokens=[9, 14, 6, 11, 8], stop_ids=(), prefill_budget=budget)
    assert eng.last_counters.mixed_steps >= 4
    pinned = sum(follows_plain(folder, p, out, tol=1e-2) for p, out in zip(prompts, outs))
    assert pinned >= 24                                   # of 48 tokens
    eng.cache.check()


def test_bfloat16_few_pages_preempt_and_recompute(model_root):
    """The bfloat16 twin of the preemption test: so few pages that requests are sent back and recomputed.  A
    recomputed prompt runs as a portion where it was decoded token by token before, so its bfloat16 logits may
    differ by rounding; every token still follows the plain implementation, and nothing is lost."""
    cfg, _, page = TINY["D"]
    folder = make_model(model_root, "D", seed=33, dtype=torch.bfloat16, std=0.08)
    prompts = [seeded_ids(n, cfg["vocab_size"], 30 + n) for n in (20, 17, 25, 9, 31, 12)]
    tight = engine(folder, "bfloat16", page_size=8, max_tokens=128, max_requests=6)    # 16 pages of 8 for six requests of ~45
    got = tight.generate(prompts, max_new_tokens=[20, 16, 12, 22, 8, 18], stop_ids=(), return_requests=True)
    assert tight.last_counters.preemptions >= 1
    assert all(r.finish_reason == "length" for r in got)
    pinned = sum(follows_plain(folder, p, r.output, tol=1e-2) for p, r in zip(prompts, got))
    assert pinned >= 48                                   # of 96 tokens
    assert sorted(tight._graphs)[-1] == 8 and len(tight._graphs) >= 3      # the decoding batch went through several graph sizes
    tight.cache.check()
    assert tight.cache.free_pages() == tight.cache.num_pages


def test_temperature_is_reproducible_independent_of_batch_and_follows_the_distribution(model_root):
    """Tiny B: three requests (7, 19, 33 tokens) cut into portions of 4, 8 or 16 beside decoded
    tokens, temperature 0.8, fixed seed."""
    from beglin_b200.sampling import uniform
    folder = make_model(model_root, "B", seed=3, dtype=torch.float32)
    prompts = [seeded_ids(n, 384, 10 + n) for n in (7, 19, 33)]
    eng = engine(folder, "float32", page_size=16)
    runs = [eng.generate(prompts, max_new_tokens=10, temperature=0.8, seed=42, stop_ids=(), prefill_budget=b)
            for b in (4, 8, 16)]
    assert runs[0] == runs[1] == runs[2]
    assert eng.generate(prompts, max_new_tokens=10, temperature=0.8, seed=43, stop_ids=()) != runs[0]
    alone = eng.generate([prompts[1]], max_new_tokens=10, temperature=0.8, seed=42, stop_ids=())[0]
    # request keys are the prompt's index: alone it is index 0, so only its own draw order matters
    assert len(alone) == 10
    for i, (p, out) in enumerate(zip(prompts, runs[0])):
        logits = plain_logits(folder, p + out)
        for k, tok in enumerate(out):
            cdf = plain.temperature_cdf(logits[len(p) + k - 1], 0.8)
            u = uniform(42, i, k)
            lo = 0.0 if tok == 0 else float(cdf[tok - 1])
            assert lo - 1e-4 <= u <= float(cdf[tok]) + 1e-4, (i, k, tok)


def test_stop_ids_and_token_limits(model_root):
    folder = make_model(model_root, "A", seed=3, dtype=torch.float32)
    eng = engine(folder, "float32")
    p = seeded_ids(6, 256, 7)
    full = eng.generate([p], max_new_tokens=12, stop_ids=())[0]
    stop = full[4]
    cut = eng.generate([p], max_new_tokens=12, stop_ids=(stop,))[0]
    assert cut == full[:full.index(stop) + 1]                      # the stop token is recorded
    assert eng.generate([p, p], max_new_tokens=[3, 0], stop_ids=()) == [full[:3], []]


def test_few_pages_preempt_and_recompute_to_the_same_tokens(model_root):
    folder = make_model(model_root, "A", seed=3, dtype=torch.float32)
    prompts = [seeded_ids(n, 256, 30 + n) for n in (20, 17, 25, 9)]
    roomy = engine(folder, "float32", max_tokens=512)
    want = roomy.generate(prompts, max_new_tokens=20, stop_ids=())
    tight = engine(folder, "float32", max_tokens=96)               # 12 pages of 8 for four requests of ~40
    got = tight.generate(prompts, max_new_tokens=20, stop_ids=(), return_requests=True)
    assert [r.output for r in got] == want
    assert tight.last_counters.preemptions >= 1
    assert all(r.finish_reason == "length" for r in got)
    tight.cache.check()
    assert tight.cache.free_pages() == tight.cache.num_pages


def test_missing_gpu_or_bad_dtype_fail_loudly(model_root):
    from beglin_b200 import Engine
    folder = make_model(model_root, "A", seed=3, dtype=torch.float32)
    with pytest.raises(RuntimeError, match="no CPU path"):
        Engine.from_folder(folder, device="cpu")
    with pytest.raises(ValueError, match="dtype"):
        Engine.from_folder(folder, dtype="float16")


def test_command_line_greedy_and_cbatch(model_root, tmp_path):
    folder = make_model(model_root, "A", seed=3, dtype=torch.float32)
    cfg, w = plain_model(folder)
    prompt = seeded_ids(40, 256, 8)
    ids = tmp_path / "prompt.i32"
    np.asarray(prompt, dtype="<i4").tofile(ids)
    env = dict(os.environ, QWEN_BASE=folder, QWEN_PROMPT=str(ids), QWEN_DTYPE="fp32", QWEN_SAFETENSORS_MAXSEQ="128",
               QWEN_PAGE_SIZE="8")
    exe = [sys.executable, os.path.join(ROOT, "bin", "qwen_infer")]
    r = subprocess.run(exe + ["greedy", "6"], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    want = plain.greedy_generate(cfg, w, prompt, 6)
    assert r.stdout.strip() == "greedy:" + "".join(f" {t}" for t in want)
    assert "[engine] arch config" in r.stderr and "NL=2" in r.stderr
    r = subprocess.run(exe + ["cbatch", "5"], env=dict(env, QWEN_CB_REQS="6", QWEN_BATCH="3", QWEN_CB_REPS="2",
                                                        QWEN_CB_PREFILL_BUDGET="8"),
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = r.stdout.strip().splitlines()
    assert len(lines) == 7 and lines[-1].startswith("agg_tok_s ") and "reps_identical 1" in lines[-1]
    plen = [min(40, 4 + (i * 13) % 37) for i in range(6)]
    maxnew = [6 + (i * 7) % 5 for i in range(6)]
    for i, line in enumerate(lines[:6]):
        head, toks = line.split(":")
        assert head == f"cbatch req{i} plen {plen[i]} maxnew {maxnew[i]} nout {maxnew[i]}"
        assert [int(t) for t in toks.split()] == plain.greedy_generate(cfg, w, prompt[:plen[i]], maxnew[i])
    # ppl: teacher-forced perplexity over the token files of <QWEN_BASE>/eval/ppl_work (one is missing, one too short)
    work = os.path.join(folder, "eval", "ppl_work")
    os.makedirs(work, exist_ok=True)
    windows = {0: seeded_ids(90, 256, 21), 2: seeded_ids(33, 256, 22), 3: [5]}
    for wi, ids_w in windows.items():
        np.asarray(ids_w, dtype="<i4").tofile(os.path.join(work, f"w{wi}.i32"))
    r = subprocess.run(exe + ["ppl", "4"], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    nll, n = 0.0, 0
    for ids_w in (windows[0], windows[2]):
        logp = torch.log_softmax(plain.forward(cfg, w, ids_w)[:-1], dim=-1)
        nll -= float(logp[torch.arange(len(ids_w) - 1), torch.tensor(ids_w[1:])].sum())
        n += len(ids_w) - 1
    word, value, word2, count = r.stdout.split()
    assert (word, word2, int(count)) == ("ppl", "tokens", n)
    assert abs(float(value) / math.exp(nll / n) - 1.0) < 1e-4
    r = subprocess.run(exe + ["greedy"], env=dict(env, QWEN_BASE=str(tmp_path)), capture_output=True, text=True, timeout=600)
    assert r.returncode == 1 and "FATAL" in r.stderr and "arch config" in r.stderr


def test_command_line_kept_variables(model_root, tmp_path):
    """QWEN_CB_MIXED=0 (prompts in steps of their own: the same tokens, stalls counted), QWEN_HF_CONFIG (the
    configuration from another place than the model folder) and QWEN_PROF=1 (time per kernel class with the
    share of the total they cover)."""
    import shutil
    folder = make_model(model_root, "A", seed=3, dtype=torch.float32)
    cfg, w = plain_model(folder)
    prompt = seeded_ids(40, 256, 8)
    ids = tmp_path / "prompt.i32"
    np.asarray(prompt, dtype="<i4").tofile(ids)
    # a folder with the weights only; its config.json lies elsewhere
    bare = tmp_path / "weights_only"
    bare.mkdir()
    shutil.copy(os.path.join(folder, "model.safetensors"), bare / "model.safetensors")
    elsewhere = tmp_path / "the_config.json"
    shutil.copy(os.path.join(folder, "config.json"), elsewhere)
    env = dict(os.environ, QWEN_BASE=str(bare), QWEN_PROMPT=str(ids), QWEN_DTYPE="fp32", QWEN_SAFETENSORS_MAXSEQ="128",
               QWEN_PAGE_SIZE="8", QWEN_HF_CONFIG=str(elsewhere))
    exe = [sys.executable, os.path.join(ROOT, "bin", "qwen_infer")]
    want = plain.greedy_generate(cfg, w, prompt, 6)
    r = subprocess.run(exe + ["greedy", "6"], env=dict(env, QWEN_PROF="1"), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout.strip().splitlines()[-1] == "greedy:" + "".join(f" {t}" for t in want)
    assert str(elsewhere) in r.stderr
    closure = [l for l in r.stderr.splitlines() if l.startswith("[prof] ctx~")]
    assert len(closure) == 1 and "closure=" in closure[0]
    share = float(closure[0].split("closure=")[1].rstrip("%"))
    assert 1.0 < share <= 100.5                       # the classes are part of the total and never more than it
    classes = [l.split()[1] for l in r.stderr.splitlines() if l.startswith("[prof]   ")]
    for name in ("emb_gather", "rmsnorm", "proj_qkv", "rope+kv_write", "attn", "proj_o", "proj_gate_up", "swiglu", "proj_down",
                 "head_gemv", "sample"):
        assert name in classes, (name, classes)
    fields = r.stdout.strip().splitlines()[0].split()
    assert fields[0] == "PROF" and fields[3] == "total_ms"
    total = float(fields[4])
    parts = sum(float(v) for v in fields[6::2])
    assert abs(parts / total * 100.0 - share) < 0.5    # the machine-readable line says the same
    r = subprocess.run(exe + ["bench", "5"], env=dict(env, QWEN_PROF="1"), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "closure=" in r.stderr and r.stdout.strip().splitlines()[-1].startswith("tok_s ")
    # the two orders of cbatch give every request the same tokens; the sequential one counts its stalls
    outs = {}
    for mixed in ("1", "0"):
        r = subprocess.run(exe + ["cbatch", "5"], env=dict(env, QWEN_CB_REQS="6", QWEN_BATCH="3", QWEN_CB_REPS="1",
                                                            QWEN_CB_PREFILL_BUDGET="8", QWEN_CB_MIXED=mixed),
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        lines = r.stdout.strip().splitlines()
        outs[mixed] = lines[:6]
        agg = lines[-1].split()
        field = lambda k: agg[agg.index(k) + 1]
        assert field("mixed") == mixed
        assert (int(field("pstall")) > 0) == (mixed == "0") and (int(field("msteps")) > 0) == (mixed == "1")
    assert outs["1"] == outs["0"]
    r = subprocess.run(exe + ["greedy"], env=dict(env, QWEN_HF_CONFIG=str(tmp_path / "missing.json")), capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 1 and "missing.json" in r.stderr and "arch config" in r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_weights_made_on_the_device_are_the_folder_of_the_same_seed(model_root, dtype):
    """`Engine.random` fills the weights on the device with the counter-based generator; the folder that the same
    seed writes on the host holds the same bits, tensor by tensor, and the two engines give the same logits bit for
    bit (so a model too large to write to disk can still be held to the plain implementation on a host)."""
    from beglin_b200 import Engine
    from beglin_b200.config import load_config
    from beglin_b200.weights import random_tensors, write_random_model
    import os
    cfg, init, page = TINY["B"]
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    arch, c = load_config(dict(cfg))
    spec = arch.build_spec(c)
    host = random_tensors(spec, 31, dtype=stored, generator="counter", **init)
    dev = random_tensors(spec, 31, dtype=stored, generator="counter", device="cuda:0", **init)
    for name in host:
        assert torch.equal(host[name], dev[name].cpu()), name
    folder = os.path.join(str(model_root), f"counter_{dtype}")
    write_random_model(folder, cfg, 31, dtype=stored, generator="counter", **init)
    ids = seeded_ids(50, cfg["vocab_size"], 2)
    a = Engine.random(cfg, 31, dtype=dtype, max_tokens=128, page_size=page, max_requests=1, **init)
    b = Engine.from_folder(folder, dtype=dtype, max_tokens=128, page_size=page, max_requests=1)
    la, lb = a.step([("r", ids, list(range(50)))]), b.step([("r", ids, list(range(50)))])
    assert torch.equal(la, lb)
    assert rel_err(la, plain_logits(folder, ids)) < (TOL_F32 if dtype == "float32" else TOL_BF16)
