"""The plain implementation checks itself (no GPU): its two attention forms agree, the loop form is
causal, windows cut what they should, rotation is a rotation, and greedy takes the first maximum."""
import math

import torch

from helpers import TINY, make_model, plain, plain_logits, plain_model, seeded_ids


def test_attention_forms_agree_and_are_causal():
    torch.manual_seed(0)
    T, nh, nkv, hd = 13, 6, 2, 16
    q = torch.randn(T, nh, hd, dtype=torch.float64)
    k = torch.randn(T, nkv, hd, dtype=torch.float64)
    v = torch.randn(T, nkv, hd, dtype=torch.float64)
    for window in (None, 4):
        a = plain.attention(q, k, v, 3, window)
        b = plain.attention_fast(q, k, v, 3, window)
        assert (a - b).abs().max() < 1e-12
    k2, v2 = k.clone(), v.clone()
    k2[7:] += 5.0
    v2[7:] -= 3.0
    assert torch.equal(plain.attention(q, k2, v2, 3)[:7], plain.attention(q, k, v, 3)[:7])
    # position 0 sees only itself: its output is v[0] of its kv head
    out = plain.attention(q, k, v, 3).reshape(T, nh, hd)
    assert (out[0, 4] - v[0, 1]).abs().max() < 1e-12
    # a window of 1 returns each position's own value
    w1 = plain.attention(q, k, v, 3, 1).reshape(T, nh, hd)
    assert (w1[:, 0] - v[:, 0]).abs().max() < 1e-12


def test_rotation_keeps_norms_and_relative_angles():
    torch.manual_seed(1)
    v = torch.randn(5, 2, 32, dtype=torch.float64)
    ang = plain.rope_angles(range(5), 32, 10000.0, torch.float64)
    r = plain.rope_split_half(v, ang)
    assert (r.norm(dim=-1) - v.norm(dim=-1)).abs().max() < 1e-12
    assert torch.equal(r[0], v[0])                       # position 0 is not rotated
    # feature i pairs with i + 16: rotating (1, 0) by the angle gives (cos, sin)
    e = torch.zeros(1, 1, 32, dtype=torch.float64)
    e[0, 0, 3] = 1.0
    # the angle is the reference's 32-bit number: 32-bit frequency times 32-bit position (qwen_infer.c:791)
    import numpy as np
    inv3 = np.float32(np.float64(np.float32(10000.0)) ** np.float64(-(np.float32(2.0) * np.float32(3)) / np.float32(32)))
    a3 = float(np.float32(7) * inv3)
    assert abs(a3 - 7 * 10000.0 ** (-(2 * 3) / 32)) < 1e-6
    r = plain.rope_split_half(e, plain.rope_angles([7], 32, 10000.0, torch.float64))
    assert abs(r[0, 0, 3] - math.cos(a3)) < 1e-12 and abs(r[0, 0, 19] - math.sin(a3)) < 1e-12


def test_rmsnorm_swiglu_and_greedy():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    y = plain.rmsnorm(x, torch.tensor([2.0, 0.5], dtype=torch.float64), 0.0)
    assert torch.allclose(y, torch.tensor([[6.0 / math.sqrt(12.5), 2.0 / math.sqrt(12.5)]], dtype=torch.float64))
    g = torch.tensor([0.0, 1.0]); u = torch.tensor([5.0, 2.0])
    assert torch.allclose(plain.swiglu(g, u), torch.tensor([0.0, 2.0 / (1 + math.exp(-1.0))]))
    assert plain.greedy_token(torch.tensor([1.0, 7.0, 7.0, 2.0])) == 1


def test_whole_model_is_causal_and_window_matters(model_root):
    folder = make_model(model_root, "C", seed=5, dtype=torch.float32)
    cfg, w = plain_model(folder)
    ids = seeded_ids(40, cfg["vocab_size"], 1)
    full = plain.forward(cfg, w, ids)
    assert torch.equal(plain.forward(cfg, w, ids[:17]), full[:17]) or \
        (plain.forward(cfg, w, ids[:17]) - full[:17]).abs().max() < 1e-12
    no_window = dict(cfg, use_sliding_window=False)
    other = plain.forward(no_window, w, ids)
    assert (other[:24] - full[:24]).abs().max() < 1e-12            # within the window nothing changes
    assert (other[30:] - full[30:]).abs().max() > 1e-9             # beyond it the window shows
    slow = plain.forward(cfg, w, ids[:20], fast=False)
    assert (slow - full[:20]).abs().max() < 1e-12


def test_greedy_generate_extends_itself(model_root):
    folder = make_model(model_root, "A", seed=2, dtype=torch.float32)
    cfg, w = plain_model(folder)
    out = plain.greedy_generate(cfg, w, [5, 9, 200], 4)
    assert len(out) == 4
    assert plain.greedy_generate(cfg, w, [5, 9, 200] + out[:2], 2) == out[2:]
