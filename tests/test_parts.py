"""Each part of a layer alone against its plain counterpart, and parts the framework does not have,
registered from here: a toy mixer with state of its own, a run order that names a layer twice, and a
layer that reads another layer's cache.  Nothing in the package is changed for them."""
import math
from dataclasses import dataclass
from typing import Dict, List

import pytest
import torch

from helpers import TINY_B, plain, rel_err, seeded_ids

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ctx_for(dtype, page=8, kv_split=64):
    from beglin_b200.csrc import ops
    from beglin_b200.parts import BuildContext
    c = BuildContext(device=DEV, compute_dtype=dtype, page_size=page, kv_split=kv_split)
    c.status = ops.new_status(DEV)
    return c


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


class OneRequest:
    """A cache manager and a step batch for a single request of a single mixer."""

    def __init__(self, need, page, pages=32):
        from beglin_b200.cache import CacheManager
        self.cache = CacheManager([need], page_size=page, num_pages=pages, max_requests=2)
        self.cache.allocate(DEV, torch.float32)
        for g in self.cache.kv_groups:
            g.device_pool.fill_(float("nan"))
        self.cache.add_request("r")

    def batch(self, tokens):
        from beglin_b200.engine.batch import Entry, StepBatch
        n = self.cache.length("r")
        plan = [("r", n + len(tokens))]
        self.cache.reserve(plan)
        b = StepBatch([Entry("r", list(tokens), [])], [n], DEV, self.cache)
        self.cache.commit(plan)
        return b


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_norm_linear_and_feed_forward_parts(dtype, tol):
    from beglin_b200.parts import Linear, NormSpec, SwiGLUSpec
    from beglin_b200.parts.mlp import SwiGLU
    from beglin_b200.parts.norm import RMSNorm
    ctx = ctx_for(dtype)
    d, im, T = 72, 136, 9
    w = 1 + rnd(d, seed=1, scale=0.1)
    norm = RMSNorm(NormSpec(size=d, eps=1e-5), {"weight": w}, ctx)
    x = rnd(T, d, seed=2).to(DEV)
    delta = rnd(T, d, seed=3).to(dtype).to(DEV)
    x0 = x.clone()
    h = norm.add_norm(x, delta)
    want_x = x0.double().cpu() + delta.double().cpu()
    assert h.dtype == dtype and (x.double().cpu() - want_x).abs().max() < 1e-6
    assert rel_err(h, plain.rmsnorm(want_x, w.double(), 1e-5)) < tol

    wt, b = rnd(50, d, seed=4, scale=0.1), rnd(50, seed=5)
    lin = Linear(wt, b, ctx)
    xin = rnd(T, d, seed=6).to(dtype).to(DEV)
    wq = wt.to(dtype).double()
    assert rel_err(lin(xin), plain.linear(xin.double().cpu(), wq, b.double())) < tol
    assert lin(xin, out_dtype=torch.float32).dtype == torch.float32

    t = {"gate_proj.weight": rnd(im, d, seed=7, scale=0.2), "up_proj.weight": rnd(im, d, seed=8, scale=0.2),
         "down_proj.weight": rnd(d, im, seed=9, scale=0.2)}
    ff = SwiGLU(SwiGLUSpec(hidden=d, intermediate=im), t, ctx)
    want = plain.mlp(xin.double().cpu(), *(t[k].to(dtype).double() for k in
                                            ("gate_proj.weight", "up_proj.weight", "down_proj.weight")))
    assert rel_err(ff.forward(xin, None), want) < tol * 2


@pytest.mark.parametrize("rows", [1, 8, 17, 64, 200])
@pytest.mark.parametrize("k,n", [(255, 176), (144, 255), (254, 720), (360, 255), (255, 1000), (4094, 48), (1536, 256),
                                 (8960, 64)])
def test_products_add_up_in_32_bit(rows, k, n):
    """A product whose halves along the inner size are large and cancel: x = [u, -u], w = [v, v + d] with small
    integers u, v and d in sixteenths, so that every product and every float sum is exact and the result is
    -sum(u d).  Whatever kernel or library routine the row count selects, one rounding to bfloat16 is all that
    may be lost; a sum of parts kept in bfloat16 on the way is wrong by whole units."""
    from beglin_b200.parts import Linear
    ctx = ctx_for(torch.bfloat16)
    g = torch.Generator().manual_seed(k * 1000 + n + rows)
    half = k // 2
    u = torch.randint(-8, 9, (rows, half), generator=g).float()
    v = torch.randint(-7, 8, (n, half), generator=g).float()
    d = torch.randint(-3, 4, (n, half), generator=g).float() / 16
    x = torch.cat([u, -u] + [torch.zeros(rows, 1)] * (k % 2), 1)          # an odd inner size: one column of zeros
    w = torch.cat([v, v + d] + [torch.ones(n, 1)] * (k % 2), 1)
    assert (w.to(torch.bfloat16).float() == w).all() and (x.to(torch.bfloat16).float() == x).all()
    want = -(u.double() @ d.double().t())
    lin = Linear(w, None, ctx)
    xin = x.to(torch.bfloat16).to(DEV)
    for out_dtype, lost in ((torch.float32, 0.0), (torch.bfloat16, 2.0 ** -8)):
        got = lin(xin, out_dtype=out_dtype).double().cpu()
        excess = ((got - want).abs() - lost * want.abs()).max()
        assert excess <= 1e-6, (out_dtype, float(excess), float(want.abs().max()))


def test_position_part_table_and_pairing():
    from beglin_b200.parts import PositionSpec
    from beglin_b200.parts.rope import shared_position
    ctx = ctx_for(torch.float32)
    spec = PositionSpec(rotary_dim=24, theta=12345.0, freq_scale=tuple(1.0 / (1 + i) for i in range(12)))
    part = shared_position(spec, ctx)
    assert shared_position(spec, ctx) is part                      # one part per distinct spec
    from beglin_b200.parts import PagedKVNeed
    one = OneRequest(PagedKVNeed(1, 24), 8)
    one.batch([1] * 5)
    b = one.batch([1, 2, 3])                                        # positions 5, 6, 7
    tab = part.table(b)
    assert part.table(b) is tab                                     # made once per step
    i = torch.arange(12, dtype=torch.float64)
    inv = 12345.0 ** (-(2 * i) / 24) / (1 + i)
    ang = torch.tensor([5.0, 6.0, 7.0], dtype=torch.float64)[:, None] * inv[None]
    assert (tab[..., 0].double().cpu() - torch.cos(ang)).abs().max() < 1e-6
    assert (tab[..., 1].double().cpu() - torch.sin(ang)).abs().max() < 1e-6


@pytest.mark.parametrize("window", [None, 5])
def test_attention_part_over_its_own_cache(window):
    """The mixer alone, a prompt in two portions and one decoded token, against the plain block."""
    from beglin_b200.parts import AttentionSpec, PositionSpec
    from beglin_b200.parts.attention import GQAAttention
    ctx = ctx_for(torch.float32, page=4, kv_split=64)
    d, nh, nkv, hd = 40, 6, 3, 16
    spec = AttentionSpec(hidden=d, n_heads=nh, n_kv_heads=nkv, head_dim=hd, qkv_bias=True, window=window,
                         position=PositionSpec(rotary_dim=hd, theta=1000.0))
    names = [r.name for r in GQAAttention.expected_tensors(spec)]
    assert "o_proj.bias" not in names and "k_proj.bias" in names
    t = {n: rnd(*r.shape, seed=20 + i, scale=0.3) for i, (n, r) in
         enumerate((r.name, r) for r in GQAAttention.expected_tensors(spec))}
    mixer = GQAAttention(spec, t, ctx)
    one = OneRequest(GQAAttention.cache_need(spec), 4)
    T = 14
    h = rnd(T, d, seed=40)
    outs = []
    for lo, hi in ((0, 9), (9, 13), (13, 14)):
        b = one.batch([0] * (hi - lo))
        outs.append(mixer.forward(h[lo:hi].to(DEV).contiguous(), b, one.cache.view(0, b)))
    got = torch.cat(outs)
    sz = dict(nh=nh, nkv=nkv, hd=hd, group=nh // nkv)
    w = {"a." + k: v.double() for k, v in t.items()}
    want = plain.attention_block(h.double(), w, "a.", sz, 1000.0, window, fast=False)
    assert rel_err(got, want) < 1e-5


# ------------------------------------------------------------------------------------------------
# Parts defined here, not in the framework.

@dataclass(frozen=True)
class DecaySpec:
    hidden: int
    decay: float
    kind: str = "toy_decay"


def register_toy_mixer():
    from beglin_b200.parts import FixedStateNeed, Linear, TensorRole, register_mixer

    @register_mixer("toy_decay")
    class DecayMixer:
        """state <- decay * state + W h_t ; out_t = state.  Its state is one vector per request."""

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
            u = self.w(h).float()
            out = torch.empty_like(u)
            slots = cache.slots.tolist()
            for i, (r0, n) in enumerate(zip(batch.row_start, batch.lens)):
                s = cache.state[slots[i]]
                for t in range(r0, r0 + n):
                    s.mul_(self.spec.decay).add_(u[t])
                    out[t] = s
            return out.to(self.ctx.compute_dtype)

    return DecayMixer


def toy_spec(cfg_json, order=None, share=False):
    """Tiny B's layers with layer 1's mixer replaced by the toy; optionally a last layer that reads
    layer 0's cache."""
    import dataclasses
    from beglin_b200.config import load_config
    from beglin_b200.parts import Stage
    arch, cfg = load_config(cfg_json)
    spec = arch.build_spec(cfg)
    l1 = spec.layers[1]
    names = {k: v for k, v in l1.names.items() if not k.startswith("mixer.")}
    names["mixer.w.weight"] = "model.layers.1.toy.w.weight"
    spec.layers[1] = l1.with_parts(mixer=DecaySpec(hidden=cfg.hidden_size, decay=0.5), names=names)
    if share:
        l2 = spec.layers[2]
        spec.layers[2] = l2.with_parts(mixer=dataclasses.replace(l2.mixer, own_kv=False))
    if order is not None:
        spec.order = [Stage(*o) if isinstance(o, tuple) else Stage(o) for o in order]
    return spec, cfg


def plain_toy_forward(cfg, w, ids, order, share):
    """The plain implementation's layers, with the toy mixer, the run order and the shared cache
    written out by hand."""
    sz = plain.sizes(cfg)
    x = plain.embed(w["model.embed_tokens.weight"], ids)
    eps, theta = cfg["rms_norm_eps"], cfg["rope_theta"]
    T = len(ids)
    kv0 = None
    for st in order:
        layer, cache = (st if isinstance(st, tuple) else (st, None))
        p = f"model.layers.{layer}."
        h = plain.rmsnorm(x, w[p + "input_layernorm.weight"], eps)
        if layer == 1:
            u = plain.linear(h, w[p + "toy.w.weight"])
            s = torch.zeros(sz["d"], dtype=torch.float64)
            a = torch.empty_like(u)
            for t in range(T):
                s = 0.5 * s + u[t]
                a[t] = s
        elif layer == 2 and share:
            ang = plain.rope_angles(range(T), sz["hd"], theta, h.dtype)
            q = plain.linear(h, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.q_proj.bias"])
            q = plain.rope_split_half(q.reshape(T, sz["nh"], sz["hd"]), ang)
            a = plain.linear(plain.attention(q, kv0[0], kv0[1], sz["group"]), w[p + "self_attn.o_proj.weight"])
        else:
            if layer == 0:
                ang = plain.rope_angles(range(T), sz["hd"], theta, h.dtype)
                k = plain.linear(h, w[p + "self_attn.k_proj.weight"], w[p + "self_attn.k_proj.bias"])
                v = plain.linear(h, w[p + "self_attn.v_proj.weight"], w[p + "self_attn.v_proj.bias"])
                kv0 = (plain.rope_split_half(k.reshape(T, sz["nkv"], sz["hd"]), ang), v.reshape(T, sz["nkv"], sz["hd"]))
            a = plain.attention_block(h, w, p + "self_attn.", sz, theta, None, fast=True)
        x = x + a
        h = plain.rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps)
        x = x + plain.mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return plain.head(x, w, cfg)


@pytest.mark.parametrize("order,share", [([0, 1, 2], False), ([0, 1, 1, 0, 2], False), ([0, 1, (2, 0)], True)])
def test_toy_mixer_run_order_and_shared_cache(order, share):
    """A mixer with state of its own is registered, built into a model and stepped; a layer runs twice
    (each run with a cache of its own); a layer reads another stage's cache.  Whole, in portions and
    token by token agree with the plain computation, for two requests side by side."""
    from beglin_b200 import Engine
    from beglin_b200.weights import TensorDict, random_tensors
    register_toy_mixer()
    spec, cfg = toy_spec(TINY_B, order, share)
    tensors = random_tensors(spec, 5, std=0.05, dtype=torch.float32)
    assert "model.layers.1.toy.w.weight" in tensors and "model.layers.1.self_attn.q_proj.weight" not in tensors
    assert ("model.layers.2.self_attn.k_proj.weight" in tensors) == (not share)
    eng = Engine(spec, TensorDict(tensors), dtype="float32", max_tokens=256, page_size=16, max_requests=3,
                 kv_split=64)
    kinds = [type(n).__name__ if n is not None else None for n in eng.model.cache_needs()]
    assert "FixedStateNeed" in kinds and (None in kinds) == share
    w = {k: v.double() for k, v in tensors.items()}
    ids = {"a": seeded_ids(40, 384, 1), "b": seeded_ids(23, 384, 2)}
    want = {r: plain_toy_forward(TINY_B, w, ids[r], order, share) for r in ids}
    whole = eng.step([("a", ids["a"], range(40)), ("b", ids["b"], range(23))], end=["a", "b"])
    assert rel_err(whole[:40], want["a"]) < 1e-4 and rel_err(whole[40:], want["b"]) < 1e-4
    # in portions and single tokens, the two requests interleaved; state and cache carry over
    got = {"a": [], "b": []}
    cuts = {"a": [0, 7, 8, 20, 21, 22, 40], "b": [0, 2, 3, 19, 23]}
    for i in range(6):
        ents = []
        for r in ("a", "b"):
            c = cuts[r]
            if i + 1 < len(c):
                ents.append((r, ids[r][c[i]:c[i + 1]], range(c[i + 1] - c[i])))
        out = eng.step(ents)
        row = 0
        for r, toks, _ in ents:
            got[r].append(out[row:row + len(toks)])
            row += len(toks)
    for r in ids:
        assert rel_err(torch.cat(got[r]), want[r]) < 1e-4, r
    # a slot that is used again starts from zero state
    eng.release("a"); eng.release("b")
    again = eng.step([("c", ids["b"], range(23))], end=["c"])
    assert rel_err(again, want["b"]) < 1e-4
