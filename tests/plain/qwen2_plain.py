"""Plain, slow implementation of the Qwen2 dense decoder, used only as the oracle of the tests.

It restates the formulas of popixoxipop-collab/beglin's `qwen_infer.c` (each function cites the
lines it restates).  That file needs Apple's Accelerate and ARM NEON headers and does not compile
whole on an x86 Linux host, but the functions of its arithmetic do when they are cut out by their
lines and given a shim of the Accelerate loops: tests/golden/make_golden.py compiles them into a
driver that runs tiny random models token by token, and tests/test_golden.py holds this file
against the driver's committed outputs (logits, greedy tokens, rotation tables up to position
32,767, frequency ratios).

Whole sequences, no cache, one function per part, plain tensor arithmetic on whatever device the
weights lie (the CPU by default; long sequences may be given weights on a GPU, in float64 still).
It shares no code with the
`beglin_b200` package: it reads the model folder with the `json` module and the `safetensors`
library and computes in float64 by default (float32 on request), so a fault of the engine's loader,
cache, batching or kernels cannot be mirrored here.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch


# ----------------------------------------------------------------------------- model folder
def read_folder(folder: str, dtype: torch.dtype = torch.float64):
    """config.json as a dict and every tensor of model.safetensors widened to `dtype`.

    The reference widens F32/F16/BF16 to fp32 on the host (safetensors_quants.c:46-61)."""
    from safetensors import safe_open

    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    weights: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name).to(dtype)
    return cfg, weights


def sizes(cfg: dict) -> dict:
    """Derived sizes as qwen_infer.c:19474-19482 derives them (head_dim may be given)."""
    d = cfg["hidden_size"]
    nh = cfg["num_attention_heads"]
    nkv = cfg["num_key_value_heads"]
    hd = cfg.get("head_dim") or d // nh
    return dict(d=d, nh=nh, nkv=nkv, hd=hd, qd=nh * hd, kvd=nkv * hd, group=nh // nkv,
                im=cfg["intermediate_size"], nl=cfg["num_hidden_layers"], vocab=cfg["vocab_size"])


def layer_window(cfg: dict, layer: int) -> Optional[int]:
    """Window of a layer from config.json's keys: with `use_sliding_window`, layers whose index is
    at least `max_window_layers` see only the last `sliding_window` positions.  The reference never
    reads these keys (full causal attention always, qwen_infer.c:1538-1543)."""
    if not cfg.get("use_sliding_window", False):
        return None
    w = cfg.get("sliding_window")
    if w is None:
        return None
    if layer >= cfg.get("max_window_layers", 0):
        return int(w)
    return None


# ----------------------------------------------------------------------------- parts
def embed(table: torch.Tensor, ids: Sequence[int]) -> torch.Tensor:
    """x = E[id], a row gather without scaling (qwen_infer.c:1438-1439, :2067)."""
    return table[torch.as_tensor(list(ids), dtype=torch.long, device=table.device)]


def rmsnorm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    """ss = sum x^2; inv = 1/sqrt(ss/n + eps); y = x*inv*g (qwen_infer.c:711-714)."""
    ss = (x * x).sum(dim=-1, keepdim=True)
    inv = 1.0 / torch.sqrt(ss / x.shape[-1] + eps)
    return x * inv * g


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[o] = bias[o] + sum_i W[o,i] x[i], W row-major [out, in] (qwen_infer.c:688-691)."""
    y = x @ w.t()
    if b is not None:
        y = y + b
    return y


def frequency_scale(cfg: dict, rot: int) -> Optional[torch.Tensor]:
    """The per-frequency ratio s_i of config.json's rope_scaling of rope_type "llama3"
    (rope_llama3_scale.h:18-28); None (all ones) without that key (qwen_infer.c:757-764).  The header
    computes in 32-bit floats throughout, and so does this, one rounded operation after the other."""
    rs = cfg.get("rope_scaling")
    if not rs:
        return None
    f32 = lambda v: torch.tensor(float(v), dtype=torch.float32)
    theta, factor, low, high = f32(cfg["rope_theta"]), f32(rs["factor"]), f32(rs["low_freq_factor"]), f32(rs["high_freq_factor"])
    orig = f32(rs["original_max_position_embeddings"])
    out = []
    for i in range(rot // 2):
        exponent = -(f32(2.0) * f32(i)) / f32(rot)
        inv = torch.pow(theta.double(), exponent.double()).float()          # powf, correctly rounded
        wavelen = (f32(2.0) * f32(math.pi)) / inv
        if wavelen > orig / low:
            out.append(f32(1.0) / factor)
        elif wavelen < orig / high:
            out.append(f32(1.0))
        else:
            smooth = (orig / wavelen - low) / (high - low)
            out.append((f32(1.0) - smooth) / factor + smooth)
    return torch.stack(out).double()


def rope_angles(positions: Sequence[int], rot: int, theta: float, dtype,
                scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """ang[p, i] = pos * inv_i, inv_i = theta^(-2i/rot) * s_i for i < rot/2 (qwen_infer.c:791-794).

    The reference makes these numbers in 32-bit: `float inv = powf(theta, -(2.0f*i)/hd); inv *= scale[i];
    float ang = pos*inv;`.  They are restated so: theta, the exponent, the frequency and the angle are
    32-bit values, `powf` correctly rounded (the 64-bit power of the 32-bit operands, rounded once).  Only
    the cosine and sine that follow are taken in `dtype`.  A 64-bit angle would be another function of the
    position: at position 4,000 the 32-bit product is 0.0002 off it."""
    i = torch.arange(rot // 2, dtype=torch.float32)
    exponent = -(2.0 * i) / torch.tensor(float(rot), dtype=torch.float32)
    inv = torch.pow(torch.tensor(float(theta), dtype=torch.float32).double(), exponent.double()).float()
    if scale is not None:
        inv = inv * scale.float()
    pos = torch.as_tensor(list(positions), dtype=torch.float32)
    return (pos[:, None] * inv[None, :]).to(dtype)            # on the CPU; `rope_split_half` moves it to its operand


def rope_split_half(v: torch.Tensor, ang: torch.Tensor) -> torch.Tensor:
    """Pairs (i, i+hd/2): v[i] = a*c - b*s; v[i+hd/2] = b*c + a*s (qwen_infer.c:782-790, the
    split-half branch).  v is [T, heads, hd], ang is [T, hd/2]."""
    half = v.shape[-1] // 2
    ang = ang.to(v.device)
    c = torch.cos(ang)[:, None, :]
    s = torch.sin(ang)[:, None, :]
    a, b = v[..., :half], v[..., half:]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group: int,
              window: Optional[int] = None, positions: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Causal grouped-query attention over a whole sequence (qwen_infer.c:1538-1543, :2127-2132):
    kvh = h / group; s_t = (q_h . K[t,kvh]) / sqrt(hd) for t <= p; softmax with the maximum
    subtracted (:715-718); o_h = sum_t p_t V[t,kvh].  With a window w only p-w < t <= p count.
    q is [T, nh, hd]; k, v are [T, nkv, hd]; the result is [T, nh*hd]."""
    T, nh, hd = q.shape
    scale = 1.0 / math.sqrt(float(hd))
    out = torch.zeros(T, nh, hd, dtype=q.dtype)
    for h in range(nh):
        kvh = h // group
        for p in range(T):
            lo = 0 if window is None else max(0, p - window + 1)
            s = (k[lo:p + 1, kvh] @ q[p, h]) * scale
            e = torch.exp(s - s.max())
            pr = e * (1.0 / e.sum())
            out[p, h] = pr @ v[lo:p + 1, kvh]
    return out.reshape(T, nh * hd)


def attention_fast(q, k, v, group, window=None, rows_at_a_time: int = 1024):
    """The same sums as `attention`, as matrix products with a mask (for long sequences), a block of
    query rows at a time so that the scores of a long sequence need not be held all at once."""
    T, nh, hd = q.shape
    scale = 1.0 / math.sqrt(float(hd))
    kk = k.repeat_interleave(group, dim=1)          # head h reads kv head h // group
    vv = v.repeat_interleave(group, dim=1)
    out = torch.empty(T, nh, hd, dtype=q.dtype, device=q.device)
    t_idx = torch.arange(T, device=q.device)[None, :]
    for lo in range(0, T, rows_at_a_time):
        hi = min(T, lo + rows_at_a_time)
        s = torch.einsum("phd,thd->hpt", q[lo:hi], kk[:hi]) * scale
        p_idx = torch.arange(lo, hi, device=q.device)[:, None]
        ok = t_idx[:, :hi] <= p_idx
        if window is not None:
            ok = ok & (t_idx[:, :hi] > p_idx - window)
        s = s.masked_fill(~ok[None], float("-inf"))
        s = s - s.max(dim=-1, keepdim=True).values
        e = torch.exp(s)
        pr = e / e.sum(dim=-1, keepdim=True)
        out[lo:hi] = torch.einsum("hpt,thd->phd", pr, vv[:hi])
    return out.reshape(T, nh * hd)


def swiglu(g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """act = (g / (1 + exp(-g))) * u (qwen_infer.c:727-733)."""
    return (g / (1.0 + torch.exp(-g))) * u


def mlp(h: torch.Tensor, wg, wu, wd) -> torch.Tensor:
    """m = Wd (silu(Wg h) * Wu h), no biases (qwen_infer.c:1560-1573)."""
    return linear(swiglu(linear(h, wg), linear(h, wu)), wd)


def attention_block(h, w: Dict[str, torch.Tensor], prefix: str, sz: dict, theta: float,
                    window: Optional[int], fast: bool, scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q,k,v with bias, RoPE on q and k after the bias, attention, o_proj without bias
    (qwen_infer.c:1451-1465, :1548)."""
    T = h.shape[0]
    q = linear(h, w[prefix + "q_proj.weight"], w.get(prefix + "q_proj.bias"))
    k = linear(h, w[prefix + "k_proj.weight"], w.get(prefix + "k_proj.bias"))
    v = linear(h, w[prefix + "v_proj.weight"], w.get(prefix + "v_proj.bias"))
    q = q.reshape(T, sz["nh"], sz["hd"])
    k = k.reshape(T, sz["nkv"], sz["hd"])
    v = v.reshape(T, sz["nkv"], sz["hd"])
    ang = rope_angles(range(T), sz["hd"], theta, h.dtype, scale)
    q = rope_split_half(q, ang)
    k = rope_split_half(k, ang)
    fn = attention_fast if fast else attention
    a = fn(q, k, v, sz["group"], window)
    return linear(a, w[prefix + "o_proj.weight"])


def decoder_layer(x, w, layer: int, cfg: dict, sz: dict, fast: bool) -> torch.Tensor:
    """h = norm(x); x += attn(h); h = norm(x); x += mlp(h) (qwen_infer.c:1447, :1552, :1556,
    :1577)."""
    p = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    h = rmsnorm(x, w[p + "input_layernorm.weight"], eps)
    x = x + attention_block(h, w, p + "self_attn.", sz, cfg["rope_theta"], layer_window(cfg, layer), fast,
                            frequency_scale(cfg, sz["hd"]))
    h = rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps)
    x = x + mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return x


def head(x, w, cfg) -> torch.Tensor:
    """Final norm, then logits = H n without bias; H is lm_head.weight when that tensor exists,
    else the embedding table (qwen_infer.c:1585-1599, :318-319)."""
    n = rmsnorm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    hw = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return linear(n, hw)


def forward(cfg: dict, w: Dict[str, torch.Tensor], ids: Sequence[int], fast: bool = True,
            layer_outputs: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence (qwen_infer.c:1435-1599)."""
    sz = sizes(cfg)
    x = embed(w["model.embed_tokens.weight"], ids)
    for layer in range(sz["nl"]):
        x = decoder_layer(x, w, layer, cfg, sz, fast)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return head(x, w, cfg)


# ----------------------------------------------------------------------------- sampling
def greedy_token(logits: torch.Tensor) -> int:
    """Index of the first maximum (qwen_infer.c:2152-2155)."""
    m = logits.max()
    return int(torch.nonzero(logits == m)[0, 0])


def greedy_generate(cfg, w, prompt: Sequence[int], n_new: int) -> List[int]:
    """The `greedy` mode's loop with a whole-sequence forward each step (qwen_infer.c:20412-20429)."""
    ids = list(prompt)
    out = []
    for _ in range(n_new):
        t = greedy_token(forward(cfg, w, ids)[-1])
        out.append(t)
        ids.append(t)
    return out


def temperature_cdf(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    """Cumulative distribution of softmax(logits / T) in index order, in float64."""
    z = logits.to(torch.float64) / temperature
    e = torch.exp(z - z.max())
    return torch.cumsum(e / e.sum(), dim=0)
