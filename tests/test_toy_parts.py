"""Two more parts that the framework does not have, registered from here and run through the engine
without a change to the package: a feed-forward that routes each token to some of several experts,
and a position encoding whose angles are not the rotary law.  They are toys, made to show that the
registries and the block take parts of another shape; neither is anyone's model."""
import dataclasses
from dataclasses import dataclass
from typing import Tuple

import pytest
import torch

from helpers import TINY_A, TINY_B, TOL_BF16, TOL_F32, plain, rel_err, seeded_ids

pytestmark = pytest.mark.gpu


# ------------------------------------------------------------------------------------------------
# A feed-forward with routing: logits = R h (float32); the top_k experts of a token share it with the
# softmax of their logits; expert e computes D_e relu(U_e h).

@dataclass(frozen=True)
class RoutedSpec:
    hidden: int
    inner: int
    n_experts: int
    top_k: int
    kind: str = "toy_routed"


def register_toy_routed():
    from beglin_b200.parts import Linear, TensorRole, register_feed_forward

    @register_feed_forward("toy_routed")
    class RoutedFeedForward:
        @staticmethod
        def expected_tensors(spec):
            roles = [TensorRole("router.weight", (spec.n_experts, spec.hidden))]
            for e in range(spec.n_experts):
                roles += [TensorRole(f"experts.{e}.up.weight", (spec.inner, spec.hidden), True, True),
                          TensorRole(f"experts.{e}.down.weight", (spec.hidden, spec.inner), True, True)]
            return roles

        def __init__(self, spec, tensors, ctx):
            self.spec, self.ctx = spec, ctx
            self.router = ctx.vector(tensors["router.weight"]).float()
            self.up = [Linear(tensors[f"experts.{e}.up.weight"], None, ctx) for e in range(spec.n_experts)]
            self.down = [Linear(tensors[f"experts.{e}.down.weight"], None, ctx) for e in range(spec.n_experts)]

        def forward(self, h, batch):
            logits = h.float() @ self.router.t()
            top, idx = torch.topk(logits, self.spec.top_k, dim=-1)
            share = torch.softmax(top, dim=-1)
            out = torch.zeros(h.shape, dtype=torch.float32, device=h.device)
            for e in range(self.spec.n_experts):
                rows, slot = torch.nonzero(idx == e, as_tuple=True)
                if rows.numel() == 0:
                    continue
                y = self.down[e](torch.relu(self.up[e](h[rows].contiguous()))).float()
                out.index_add_(0, rows, y * share[rows, slot][:, None])
            return out.to(self.ctx.compute_dtype)

    return RoutedFeedForward


CHOSEN = set()          # the experts that plain_routed has sent a token to


def plain_routed(h, w, p, spec):
    logits = plain.linear(h, w[p + "router.weight"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        top, idx = torch.topk(logits[t], spec.top_k)
        share = torch.softmax(top, dim=-1)
        CHOSEN.update(idx.tolist())
        for s, e in zip(share, idx.tolist()):
            u = torch.relu(plain.linear(h[t:t + 1], w[p + f"experts.{e}.up.weight"]))
            out[t] += s * plain.linear(u, w[p + f"experts.{e}.down.weight"])[0]
    return out


# ------------------------------------------------------------------------------------------------
# A position encoding with angles pos * step * (i + 1) + phase_i over the first `rotary_dim` features
# of a head: a table of (cos, sin) per row of the step is all that the attention part asks of it.

@dataclass(frozen=True)
class PhaseSpec:
    rotary_dim: int
    step: float
    phase: Tuple[float, ...]
    kind: str = "toy_phase"


def register_toy_phase():
    from beglin_b200.parts import register_position

    @register_position("toy_phase")
    class PhasePosition:
        def __init__(self, spec, ctx):
            self.spec, self.ctx = spec, ctx
            self.rotary_dim, self.interleaved = spec.rotary_dim, False
            half = spec.rotary_dim // 2
            self.freq = (torch.arange(1, half + 1, dtype=torch.float32) * spec.step).to(ctx.device)
            self.phase = torch.tensor(spec.phase, dtype=torch.float32, device=ctx.device)

        def table(self, batch):
            key = ("toy_phase", id(self))
            t = batch.scratch.get(key)
            if t is None:
                ang = batch.positions.float()[:, None] * self.freq[None, :] + self.phase[None, :]
                t = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).contiguous()
                batch.scratch[key] = t
            return t

    return PhasePosition


def plain_phase_attention(h, w, p, sz, spec):
    T = h.shape[0]
    half = spec.rotary_dim // 2
    ang = (torch.arange(T, dtype=torch.float64)[:, None] * (torch.arange(1, half + 1, dtype=torch.float64) * spec.step)[None, :]
           + torch.tensor(spec.phase, dtype=torch.float64)[None, :])

    def turn(x, heads):
        x = x.reshape(T, heads, sz["hd"])
        return torch.cat([plain.rope_split_half(x[..., :spec.rotary_dim], ang), x[..., spec.rotary_dim:]], dim=-1)
    q = turn(plain.linear(h, w[p + "q_proj.weight"], w[p + "q_proj.bias"]), sz["nh"])
    k = turn(plain.linear(h, w[p + "k_proj.weight"], w[p + "k_proj.bias"]), sz["nkv"])
    v = plain.linear(h, w[p + "v_proj.weight"], w[p + "v_proj.bias"]).reshape(T, sz["nkv"], sz["hd"])
    return plain.linear(plain.attention_fast(q, k, v, sz["group"]), w[p + "o_proj.weight"])


# ------------------------------------------------------------------------------------------------

def plain_forward(cfg, w, ids, routed=None, phase=None):
    """The plain implementation's layers with the toy parts in the places the test's spec puts them:
    `routed` maps a layer to its RoutedSpec, `phase` a layer to its PhaseSpec."""
    sz = plain.sizes(cfg)
    x = plain.embed(w["model.embed_tokens.weight"], ids)
    eps = cfg["rms_norm_eps"]
    for layer in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        h = plain.rmsnorm(x, w[p + "input_layernorm.weight"], eps)
        if phase and layer in phase:
            x = x + plain_phase_attention(h, w, p + "self_attn.", sz, phase[layer])
        else:
            x = x + plain.attention_block(h, w, p + "self_attn.", sz, cfg["rope_theta"], None, fast=True)
        h = plain.rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps)
        if routed and layer in routed:
            x = x + plain_routed(h, w, p + "toy.", routed[layer])
        else:
            x = x + plain.mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return plain.head(x, w, cfg)


def whole_and_cut(eng, ids, want, tol):
    """Two requests whole in one step, then in interleaved portions down to single tokens."""
    na, nb = len(ids["a"]), len(ids["b"])
    whole = eng.step([("a", ids["a"], range(na)), ("b", ids["b"], range(nb))], end=["a", "b"])
    assert rel_err(whole[:na], want["a"]) < tol and rel_err(whole[na:], want["b"]) < tol
    cuts = {"a": [0, 9, 10, 11, 30, na], "b": [0, 2, 17, 18, nb]}
    got = {"a": [], "b": []}
    for i in range(5):
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
        assert rel_err(torch.cat(got[r]), want[r]) < tol, r


def test_toy_routed_feed_forward_in_one_layer():
    """Layer 1 of three gets the routed feed-forward; the others keep the dense one.  Every expert is
    chosen by some token, and the engine agrees with the plain computation whole and in portions."""
    from beglin_b200 import Engine
    from beglin_b200.config import load_config
    from beglin_b200.weights import TensorDict, random_tensors
    register_toy_routed()
    arch, cfg = load_config(TINY_B)
    spec = arch.build_spec(cfg)
    rs = RoutedSpec(hidden=cfg.hidden_size, inner=40, n_experts=5, top_k=2)
    l1 = spec.layers[1]
    names = {k: v for k, v in l1.names.items() if not k.startswith("feed_forward.")}
    roles = register_toy_routed().expected_tensors(rs)
    names.update({"feed_forward." + r.name: "model.layers.1.toy." + r.name for r in roles})
    spec.layers[1] = l1.with_parts(feed_forward=rs, names=names)
    tensors = random_tensors(spec, 11, std=0.05, dtype=torch.float32)
    assert "model.layers.1.mlp.gate_proj.weight" not in tensors and "model.layers.1.toy.experts.4.down.weight" in tensors
    # a router that spreads the tokens: larger logits than the random draw gives
    tensors["model.layers.1.toy.router.weight"] = tensors["model.layers.1.toy.router.weight"] * 8.0
    eng = Engine(spec, TensorDict(tensors), dtype="float32", max_tokens=256, page_size=16, max_requests=3, kv_split=64)
    w = {k: v.double() for k, v in tensors.items()}
    ids = {"a": seeded_ids(41, 384, 3), "b": seeded_ids(22, 384, 4)}
    CHOSEN.clear()
    want = {r: plain_forward(TINY_B, w, ids[r], routed={1: rs}) for r in ids}
    assert CHOSEN == set(range(rs.n_experts))
    whole_and_cut(eng, ids, want, TOL_F32)


@pytest.mark.parametrize("dtype,tol", [("float32", TOL_F32), ("bfloat16", TOL_BF16)])
def test_toy_position_encoding_in_one_layer(dtype, tol):
    """Layer 0 of two turns only the first 8 of its 16 features per head, by angles with a phase; layer 1
    keeps the rotary law.  The two encodings live side by side in one model."""
    from beglin_b200 import Engine
    from beglin_b200.config import load_config
    from beglin_b200.weights import TensorDict, random_tensors
    register_toy_phase()
    arch, cfg = load_config(TINY_A)
    spec = arch.build_spec(cfg)
    ps = PhaseSpec(rotary_dim=8, step=0.37, phase=(0.1, -0.7, 1.9, 0.4))
    l0 = spec.layers[0]
    spec.layers[0] = l0.with_parts(mixer=dataclasses.replace(l0.mixer, position=ps))
    tensors = random_tensors(spec, 12, std=0.08, bias_std=0.05, dtype=torch.float32)
    if dtype == "bfloat16":
        tensors = {k: v.to(torch.bfloat16) for k, v in tensors.items()}
    eng = Engine(spec, TensorDict(tensors), dtype=dtype, max_tokens=256, page_size=8, max_requests=3, kv_split=64)
    w = {k: v.double() for k, v in tensors.items()}
    ids = {"a": seeded_ids(37, 256, 5), "b": seeded_ids(21, 256, 6)}
    want = {r: plain_forward(TINY_A, w, ids[r], phase={0: ps}) for r in ids}
    whole_and_cut(eng, ids, want, tol)


# ------------------------------------------------------------------------------------------------
# Two block arrangements the framework does not have.  "toy_parallel": one norm, the mixer and the
# feed-forward both read it, x += mixer(h) + feed_forward(h): three slots.  "toy_ff_post": no mixer at
# all and the norm AFTER the part, x += norm(feed_forward(x_bf)): two slots, one of them a norm that is
# applied to the part's result instead of to the stream.

def register_toy_blocks():
    from beglin_b200.parts import register_block

    @register_block("toy_parallel")
    class ParallelBlock:
        SLOTS = (("norm", "norm"), ("mixer", "mixer"), ("feed_forward", "feed_forward"))

        def __init__(self, norm, mixer, feed_forward):
            self.norm, self.mixer, self.feed_forward = norm, mixer, feed_forward

        def forward(self, stream, batch, cache):
            h = self.norm.add_norm(stream.x, stream.pending)      # adds what is owed, then norms
            stream.pending = stream.ssq = None
            a = self.mixer.forward(h, batch, cache)
            m = self.feed_forward.forward(h, batch)

            def whole(t):                                          # a product may return partial sums over ranges of K
                return (t.sum(dim=0) if t.dim() == 3 else t).float()
            stream.owe(whole(a) + whole(m))

    @register_block("toy_ff_post")
    class FeedForwardPostNormBlock:
        SLOTS = (("feed_forward", "feed_forward"), ("post_norm", "norm"))

        def __init__(self, feed_forward, post_norm):
            self.feed_forward, self.post_norm = feed_forward, post_norm

        def forward(self, stream, batch, cache):
            assert cache is None                                   # a layer without a mixer has no cache
            if stream.pending is not None:
                p = stream.pending
                stream.x += (p.sum(dim=0) if p.dim() == 3 else p).float()
                stream.pending = stream.ssq = None
            m = self.feed_forward.forward(stream.x.to(self.feed_forward.ctx.compute_dtype), batch)
            m = (m.sum(dim=0) if m.dim() == 3 else m).float().contiguous()
            stream.owe(self.post_norm.add_norm(m, None, update=False).float())


def plain_toy_blocks_forward(cfg, w, ids):
    """Layer 0: the reference's block.  Layer 1: parallel.  Layer 2: feed-forward only, norm after it."""
    sz = plain.sizes(cfg)
    eps, theta = cfg["rms_norm_eps"], cfg["rope_theta"]
    x = plain.embed(w["model.embed_tokens.weight"], ids)
    p = "model.layers.0."
    h = plain.rmsnorm(x, w[p + "input_layernorm.weight"], eps)
    x = x + plain.attention_block(h, w, p + "self_attn.", sz, theta, None, fast=True)
    h = plain.rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps)
    x = x + plain.mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    p = "model.layers.1."
    h = plain.rmsnorm(x, w[p + "input_layernorm.weight"], eps)
    x = x + plain.attention_block(h, w, p + "self_attn.", sz, theta, None, fast=True) \
        + plain.mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    p = "model.layers.2."
    m = plain.mlp(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    x = x + plain.rmsnorm(m, w[p + "after.weight"], eps)
    return plain.head(x, w, cfg)


def test_toy_blocks_with_other_slots():
    """A block kind declares its slots; the loader asks exactly those parts for their tensors and the model
    builds exactly those parts.  Three layers with three arrangements (four slots, three, two; one without a
    mixer and therefore without a cache) run whole and cut against the plain computation written out by hand."""
    from beglin_b200 import Engine
    from beglin_b200.config import load_config
    from beglin_b200.parts import LayerSpec
    from beglin_b200.weights import TensorDict, expected_tensors, random_tensors
    register_toy_blocks()
    arch, cfg = load_config(TINY_B)
    spec = arch.build_spec(cfg)
    l1, l2 = spec.layers[1], spec.layers[2]
    names1 = {k: v for k, v in l1.names.items() if not k.endswith("_norm.weight")}
    names1["norm.weight"] = "model.layers.1.input_layernorm.weight"
    spec.layers[1] = LayerSpec({"norm": l1.mixer_norm, "mixer": l1.mixer, "feed_forward": l1.feed_forward},
                               names1, block="toy_parallel")
    names2 = {k: v for k, v in l2.names.items() if k.startswith("feed_forward.")}
    names2["post_norm.weight"] = "model.layers.2.after.weight"
    spec.layers[2] = LayerSpec({"feed_forward": l2.feed_forward, "post_norm": l2.feed_forward_norm}, names2,
                               block="toy_ff_post")
    wanted = set(expected_tensors(spec))
    assert "model.layers.1.post_attention_layernorm.weight" not in wanted
    assert "model.layers.2.after.weight" in wanted and not any(".2.self_attn." in n for n in wanted)
    with pytest.raises(KeyError, match="lacks"):
        expected_tensors(dataclasses.replace(spec, layers=[spec.layers[0], spec.layers[1],
                                                           LayerSpec({"feed_forward": l2.feed_forward}, names2, "toy_ff_post")]))
    tensors = random_tensors(spec, 13, std=0.05, bias_std=0.05, dtype=torch.float32)
    eng = Engine(spec, TensorDict(tensors), dtype="float32", max_tokens=256, page_size=16, max_requests=3, kv_split=64)
    assert [type(n).__name__ if n is not None else None for n in eng.model.cache_needs()] == ["PagedKVNeed", "PagedKVNeed", None]
    w = {k: v.double() for k, v in tensors.items()}
    ids = {"a": seeded_ids(41, 384, 7), "b": seeded_ids(22, 384, 8)}
    want = {r: plain_toy_blocks_forward(TINY_B, w, ids[r]) for r in ids}
    whole_and_cut(eng, ids, want, TOL_F32)


# ------------------------------------------------------------------------------------------------
# The two ends of the model are the spec's business too: a scale on the embedded rows, a bias on the logits and a
# cap c * tanh(logits / c).  The architecture here has none of them; a spec with all three is stepped whole and cut.
def plain_ends_forward(cfg, w, ids, scale, cap):
    sz = plain.sizes(cfg)
    x = plain.embed(w["model.embed_tokens.weight"], ids) * scale
    eps = cfg["rms_norm_eps"]
    for layer in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        h = plain.rmsnorm(x, w[p + "input_layernorm.weight"], eps)
        x = x + plain.attention_block(h, w, p + "self_attn.", sz, cfg["rope_theta"], None, fast=True)
        h = plain.rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps)
        x = x + plain.mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    logits = plain.head(x, w, cfg) + w["toy.head_bias"]
    return cap * torch.tanh(logits / cap)


@pytest.mark.parametrize("dtype,tol", [("float32", TOL_F32), ("bfloat16", TOL_BF16)])
def test_scaled_embedding_head_bias_and_logit_cap(dtype, tol):
    from beglin_b200 import Engine
    from beglin_b200.config import load_config
    from beglin_b200.weights import TensorDict, expected_tensors, random_tensors
    arch, cfg = load_config(TINY_B)
    spec = dataclasses.replace(arch.build_spec(cfg), embed_scale=3.0, head_bias_name="toy.head_bias", logit_softcap=2.5)
    assert expected_tensors(spec)["toy.head_bias"].shape == (384,)
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    tensors = random_tensors(spec, 17, std=0.05, bias_std=0.5, dtype=stored)
    eng = Engine(spec, TensorDict(tensors), dtype=dtype, max_tokens=256, page_size=16, max_requests=3, kv_split=64)
    w = {k: v.double() for k, v in tensors.items()}
    ids = {"a": seeded_ids(41, 384, 7), "b": seeded_ids(22, 384, 8)}
    want = {r: plain_ends_forward(TINY_B, w, ids[r], 3.0, 2.5) for r in ids}
    assert float(want["a"].abs().max()) > 1.5                       # the cap bites
    whole_and_cut(eng, ids, want, tol)
    plainer = Engine(arch.build_spec(cfg), TensorDict({k: v for k, v in tensors.items() if k != "toy.head_bias"}), dtype=dtype,
                     max_tokens=256, page_size=16, max_requests=1)
    base = plainer.step([("a", ids["a"], range(41))])
    assert rel_err(base, want["a"]) > 0.1                           # and the three options are what makes the difference
