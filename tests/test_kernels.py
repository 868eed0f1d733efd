"""Each CUDA kernel alone against a plain PyTorch reference of the same operation, at sizes other
than the engine's: head sizes in steps of 16, odd numbers of heads and groups, widths that are no
powers of two, pages in shuffled order with poisoned free pages."""
import math

import pytest
import torch

from helpers import plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from beglin_b200.csrc import ops as o
    o.lib()
    return o


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_gather(ops, dtype):
    table = rnd(301, 72, dtype=dtype, seed=1)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32, device=DEV)
    out = torch.full((5, 72), float("nan"), device=DEV)
    status = ops.new_status(DEV)
    ops.embed_gather(table, ids, out, status)
    assert torch.equal(out, table.float()[ids.long()])
    ops.raise_on_status(status)
    bad = torch.tensor([3, 301], dtype=torch.int32, device=DEV)
    out2 = torch.empty((2, 72), device=DEV)
    ops.embed_gather(table, bad, out2, status)
    with pytest.raises(ops.KernelError, match="vocabulary"):
        ops.raise_on_status(status)
    assert torch.equal(out2[1], torch.zeros(72, device=DEV))


@pytest.mark.parametrize("d", [64, 1536, 100, 5000, 12288, 16392])      # 12,288: a row of exactly 48 KB in shared memory
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(ops, d, out_dtype):
    T, eps = 7, 1e-5
    x = rnd(T, d, seed=2)
    delta = rnd(T, d, dtype=out_dtype, seed=3)
    w = (1 + 0.1 * rnd(d, seed=4)).to(out_dtype if out_dtype == torch.bfloat16 else torch.float32)
    want_x = x.double() + delta.double()
    want = plain.rmsnorm(want_x, w.double(), eps)
    x1 = x.clone()
    out = torch.empty((T, d), dtype=out_dtype, device=DEV)
    ops.add_rmsnorm(x1, delta, w, eps, out)
    assert (x1.double() - want_x).abs().max() < 1e-6
    tol = 1e-5 if out_dtype == torch.float32 else 1e-2
    assert (out.double() - want).abs().max() < tol * want.abs().max()
    # without an addend x is left alone; with rows only those rows are normed and x is not updated
    x2 = x.clone()
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    out2 = torch.empty((3, d), dtype=out_dtype, device=DEV)
    ops.add_rmsnorm(x2, delta, w, eps, out2, rows=rows, update=False)
    assert torch.equal(x2, x)
    assert torch.equal(out2, out[rows.long()])
    # the addend as partial sums of a split-K product: added in index order, same result
    x4 = x.clone()
    parts = torch.stack([0.5 * delta.float(), 0.25 * delta.float(), 0.25 * delta.float()]).contiguous()
    out4 = torch.empty((T, d), dtype=out_dtype, device=DEV)
    ops.add_rmsnorm(x4, parts, w, eps, out4)
    assert (x4.double() - want_x).abs().max() < 1e-6
    assert (out4.double() - want).abs().max() < tol * want.abs().max()
    out3 = torch.empty((T, d), dtype=out_dtype, device=DEV)
    ops.add_rmsnorm(x2, None, w, eps, out3)
    want3 = plain.rmsnorm(x.double(), w.double(), eps)
    assert (out3.double() - want3).abs().max() < tol * want3.abs().max() and torch.equal(x2, x)


@pytest.mark.parametrize("T,d,parts", [(64, 1536, 13), (32, 3584, 5), (20, 5120, 7), (17, 896, 2), (3, 8192, 4), (40, 24, 3)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm_of_partial_sums_for_few_rows(ops, T, d, parts, out_dtype):
    """The addend as float partial sums of a split-K product, for the row counts of decoding steps of 17 to 64
    tokens: bfloat16 results come from clusters of 2, 4 or 8 CTAs per row (every cluster size is met here, and a row
    shorter than the cluster), float results from the block per row; with the stream updated, and with rows picked by
    a list and the stream left alone."""
    eps = 1e-6
    x = rnd(T, d, seed=T)
    ps = torch.stack([rnd(T, d, seed=100 + i, scale=0.5) for i in range(parts)]).contiguous()
    w = (1 + 0.1 * rnd(d, seed=4)).to(out_dtype if out_dtype == torch.bfloat16 else torch.float32)
    want_x = x.double() + ps.double().sum(0)
    want = plain.rmsnorm(want_x, w.double(), eps)
    tol = 1e-5 if out_dtype == torch.float32 else 1e-2
    x1 = x.clone()
    out = torch.full((T, d), float("nan"), dtype=out_dtype, device=DEV)
    ops.add_rmsnorm(x1, ps, w, eps, out)
    assert (x1.double() - want_x).abs().max() < 1e-5
    assert (out.double() - want).abs().max() < tol * want.abs().max()
    picked = [T - 1, 0, T // 2, T - 1]
    rows = torch.tensor(picked, dtype=torch.int32, device=DEV)
    x2 = x.clone()
    out2 = torch.full((len(picked), d), float("nan"), dtype=out_dtype, device=DEV)
    ops.add_rmsnorm(x2, ps, w, eps, out2, rows=rows, update=False)
    assert torch.equal(x2, x)
    assert torch.equal(out2, out[rows.long()])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu(ops, dtype):
    gu = rnd(5, 2 * 203, dtype=dtype, seed=5, scale=3.0)
    out = torch.empty((5, 203), dtype=dtype, device=DEV)
    ops.swiglu(gu, out)
    want = plain.swiglu(gu[:, :203].double(), gu[:, 203:].double())
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    assert (out.double() - want).abs().max() <= tol * want.abs().max()
    parts = torch.stack([0.5 * gu.float(), 0.5 * gu.float()]).contiguous()
    out2 = torch.empty((5, 203), dtype=dtype, device=DEV)
    ops.swiglu(parts, out2)
    assert (out2.double() - want).abs().max() <= tol * want.abs().max()


@pytest.mark.parametrize("dtype,block,im", [(torch.float32, 64, 192), (torch.bfloat16, 64, 128), (torch.float32, 5, 35),
                                            (torch.bfloat16, 8, 200)])
def test_swiglu_interleaved_blocks(ops, dtype, block, im):
    """Columns in blocks: gate, up, gate, up, ... (the layout of the fused product's weight)."""
    g, u = rnd(7, im, dtype=dtype, seed=21, scale=2.0), rnd(7, im, dtype=dtype, seed=22, scale=2.0)
    gu = torch.stack([g.reshape(7, im // block, block), u.reshape(7, im // block, block)], dim=2).reshape(7, 2 * im).contiguous()
    want = plain.swiglu(g.double(), u.double())
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    out = torch.empty((7, im), dtype=dtype, device=DEV)
    ops.swiglu(gu, out, block)
    assert (out.double() - want).abs().max() <= tol * want.abs().max()
    parts = torch.stack([0.25 * gu.float(), 0.75 * gu.float()]).contiguous()
    out2 = torch.empty((7, im), dtype=dtype, device=DEV)
    ops.swiglu(parts, out2, block)
    assert (out2.double() - want).abs().max() <= tol * want.abs().max()


def test_gemm_f32_is_true_float_and_row_invariant(ops):
    M, N, K = 37, 203, 301
    a = rnd(M, K, seed=6)
    w = rnd(N, K, seed=7)
    b = rnd(N, seed=8)
    out = torch.empty((M, N), device=DEV)
    ops.gemm_f32_nt(a, w, b, out)
    want = a.double() @ w.double().t() + b.double()
    assert (out.double() - want).abs().max() < 2e-6 * want.abs().max() * math.sqrt(K)
    # a value that tf32 (10 mantissa bits) cannot hold must survive
    a2 = torch.zeros((1, 16), device=DEV); w2 = torch.zeros((1, 16), device=DEV)
    a2[0, 0] = 1.0 + 2.0 ** -20; w2[0, 0] = 1.0
    o2 = torch.empty((1, 1), device=DEV)
    ops.gemm_f32_nt(a2, w2, None, o2)
    assert float(o2) == 1.0 + 2.0 ** -20
    # a row's result does not depend on the rows around it
    one = torch.empty((1, N), device=DEV)
    ops.gemm_f32_nt(a[11:12].contiguous(), w, b, one)
    assert torch.equal(one[0], out[11])
    acc = out.clone()
    ops.gemm_f32_nt(a, w, None, acc, accumulate=True)
    assert (acc.double() - (2 * want - b.double())).abs().max() < 1e-4


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd,rot", [(48, 32), (64, 64), (128, 128)])      # partial rotary; whole heads (16-byte path)
def test_rope_table_and_kv_append(ops, interleaved, dtype, hd, rot):
    nh, nkv, page, T = 3, 2, 8, 6
    theta = 50000.0
    positions = torch.tensor([9, 10, 11, 0, 40, 7], dtype=torch.int32, device=DEV)
    row_req = torch.tensor([0, 0, 0, 1, 2, 1], dtype=torch.int32, device=DEV)
    i = torch.arange(rot // 2, dtype=torch.float64)
    inv = torch.pow(torch.tensor(theta, dtype=torch.float64), -(2 * i) / rot).float().to(DEV)
    table = torch.empty((T, rot // 2, 2), device=DEV)
    ops.rope_table(positions, inv, table)
    ang = positions.double()[:, None].cpu() * inv.double().cpu()[None, :]
    assert (table[..., 0].cpu().double() - torch.cos(ang)).abs().max() < 2e-5   # float angle at position 40
    assert (table[..., 1].cpu().double() - torch.sin(ang)).abs().max() < 2e-5
    width = (nh + 2 * nkv) * hd
    qkv = rnd(T, width, dtype=dtype, seed=9)
    orig = qkv.clone()
    n_pages = 10
    bt = torch.full((3, 8), -1, dtype=torch.int32, device=DEV)
    bt[0, :2] = torch.tensor([4, 7]); bt[1, :1] = torch.tensor([2]); bt[2, :6] = torch.tensor([9, 0, 1, 3, 5, 6])
    pool = torch.full((n_pages, 2, nkv, page, hd), float("nan"), dtype=dtype, device=DEV)
    status = ops.new_status(DEV)
    # the rows arrive as three partial sums of a split-K product (float) or as one tensor
    if dtype == torch.float32:
        parts = torch.stack([0.25 * qkv, 0.5 * qkv, 0.25 * qkv]).contiguous()
    else:
        parts = qkv
    q_out = torch.full((T, nh * hd), float("nan"), dtype=dtype, device=DEV)
    ops.rope_kv_append(parts, q_out, T, nh, nkv, hd, rot, interleaved, table, positions, row_req, bt, pool, page, status)
    ops.raise_on_status(status)

    def rotate(v, t):        # v [heads, hd] float64
        c, s = table[t, :, 0].double().cpu(), table[t, :, 1].double().cpu()
        out = v.clone()
        if interleaved:
            a, b = v[:, 0:rot:2], v[:, 1:rot:2]
            out[:, 0:rot:2] = a * c - b * s
            out[:, 1:rot:2] = b * c + a * s
        else:
            a, b = v[:, :rot // 2], v[:, rot // 2:rot]
            out[:, :rot // 2] = a * c - b * s
            out[:, rot // 2:rot] = b * c + a * s
        return out

    tol = 1e-6 if dtype == torch.float32 else 2e-2
    written = set()
    for t in range(T):
        o = orig[t].double().cpu()
        q = rotate(o[:nh * hd].reshape(nh, hd), t)
        k = rotate(o[nh * hd:(nh + nkv) * hd].reshape(nkv, hd), t)
        v = o[(nh + nkv) * hd:].reshape(nkv, hd)
        assert (q_out[t].double().cpu().reshape(nh, hd) - q).abs().max() < tol * 4
        p = int(positions[t]); pg = int(bt[int(row_req[t]), p // page]); sl = p % page
        assert (pool[pg, 0, :, sl].double().cpu() - k).abs().max() < tol * 4
        assert (pool[pg, 1, :, sl].double().cpu() - v).abs().max() < tol * 4
        written.add((pg, sl))
        assert torch.equal(qkv[t], orig[t])                             # the source rows are not touched
    finite = torch.isfinite(pool[:, 0, 0, :, 0].float()).cpu()
    assert {(int(a), int(b)) for a, b in finite.nonzero()} == written   # nothing else was written
    # a page outside the pool is recorded, not written
    bt[1, 0] = 99
    ops.rope_kv_append(orig.clone(), q_out, T, nh, nkv, hd, rot, interleaved, table, positions, row_req, bt, pool, page, status)
    with pytest.raises(ops.KernelError, match="page"):
        ops.raise_on_status(status)


@pytest.mark.gpu
@pytest.mark.parametrize("nh,nkv,hd,dtype", [(5, 1, 48, torch.float32), (40, 4, 256, torch.float32), (48, 3, 256, torch.float32),
                                             (64, 4, 256, torch.float32), (200, 4, 256, torch.float32), (12, 2, 128, torch.bfloat16), (48, 3, 256, torch.bfloat16)])
def test_rope_and_kv_append_of_many_tokens(ops, nh, nkv, hd, dtype):
    """A portion of 100 tokens (one block per token, its q/k/v row staged in shared memory): rows of up to 48 KB (and of 48 KB to the byte), rows that
    need the larger shared-memory carve-out (55 and 73 KB) and a row that fits no SM (213 KB: head by head)."""
    T, page, rot = 100, 16, hd
    positions = torch.arange(3, 3 + T, dtype=torch.int32, device=DEV)
    row_req = torch.zeros(T, dtype=torch.int32, device=DEV)
    inv = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -(2 * torch.arange(rot // 2, dtype=torch.float64)) / rot).float().to(DEV)
    table = torch.empty((T, rot // 2, 2), device=DEV)
    ops.rope_table(positions, inv, table)
    qkv = rnd(T, (nh + 2 * nkv) * hd, dtype=dtype, seed=nh)
    n_pages = 9
    bt = torch.tensor([[5, 2, 8, 0, 7, 3, 1, -1]], dtype=torch.int32, device=DEV)       # positions 3..102 lie in 7 pages
    pool = torch.full((n_pages, 2, nkv, page, hd), float("nan"), dtype=dtype, device=DEV)
    q_out = torch.full((T, nh * hd), float("nan"), dtype=dtype, device=DEV)
    status = ops.new_status(DEV)
    ops.rope_kv_append(qkv, q_out, T, nh, nkv, hd, rot, False, table, positions, row_req, bt, pool, page, status)
    ops.raise_on_status(status)
    c, s_ = table[..., 0].double().cpu()[:, None, :], table[..., 1].double().cpu()[:, None, :]
    o = qkv.double().cpu().reshape(T, nh + 2 * nkv, hd)

    def rotate(v):                                                     # v [T, heads, hd]
        a, b = v[..., :hd // 2], v[..., hd // 2:]
        return torch.cat([a * c - b * s_, b * c + a * s_], dim=-1)

    tol = 4e-6 if dtype == torch.float32 else 8e-2
    assert (q_out.double().cpu().reshape(T, nh, hd) - rotate(o[:, :nh])).abs().max() < tol
    k, v = rotate(o[:, nh:nh + nkv]), o[:, nh + nkv:]
    for t in range(T):
        p_ = 3 + t
        pg, sl = int(bt[0, p_ // page]), p_ % page
        assert (pool[pg, 0, :, sl].double().cpu() - k[t]).abs().max() < tol
        assert (pool[pg, 1, :, sl].double().cpu() - v[t]).abs().max() < tol
    held = torch.isfinite(pool[:, 0, 0, :, 0].float()).cpu().sum()
    assert int(held) == T                                              # nothing else was written


def _attention_case(ops, nh, nkv, hd, page, dtype, window, seed, split=64, prefer="generic", decode_only=False,
                    long=False):
    """Three requests in one step: a long prompt portion on top of earlier context, a decoded token
    far into a long context, and a fresh short prompt.  Pages are handed out in shuffled order and
    everything not held is poison."""
    torch.manual_seed(seed)
    group = nh // nkv
    ctx = [(37, 21), (150, 1), (0, 5)]               # (positions already in the cache, new rows)
    if decode_only:
        ctx = [(37, 1), (150, 1), (0, 1), (63, 1), (64, 1), (127, 1), (200, 1)]
    if long:                                         # many key tiles: every pipeline stage is reused several times
        ctx = [(517, 90), (1000, 1), (0, 333)] if not decode_only else [(517, 1), (1000, 1), (0, 1), (2100, 1), (4400, 1)]
    if long == "wide":                               # thousands of keys: the tcgen05 kernel in either arrangement of its tiles
        ctx = [(6144, 2048), (5300, 1), (0, 333)]
    total = [c + n for c, n in ctx]
    n_pages_each = [-(-t // page) for t in total]
    n_pages = sum(n_pages_each) + 5
    perm = torch.randperm(n_pages).tolist()
    max_pages = max(n_pages_each) + 2
    bt = torch.full((len(ctx), max_pages), -1, dtype=torch.int32)
    pool = torch.full((n_pages, 2, nkv, page, hd), float("nan"), dtype=dtype)
    ks, vs, qs = [], [], []
    it = iter(perm)
    for r, t in enumerate(total):
        k = torch.randn(t, nkv, hd) * 0.7
        v = torch.randn(t, nkv, hd)
        k, v = k.to(dtype), v.to(dtype)
        ks.append(k); vs.append(v)
        for pi in range(n_pages_each[r]):
            pg = next(it)
            bt[r, pi] = pg
            n = min(page, t - pi * page)
            pool[pg, 0, :, :n] = k[pi * page:pi * page + n].transpose(0, 1)
            pool[pg, 1, :, :n] = v[pi * page:pi * page + n].transpose(0, 1)
    rows = sum(n for _, n in ctx)
    q = (torch.randn(rows, nh, hd) * 0.7).to(dtype)
    # make one far key stand out for the decoded token: its score dominates unless it is missed
    far, far_row = 3, (1 if decode_only else ctx[0][1])
    q[far_row, :, :] = 0; q[far_row, :, 0] = 8.0
    ks[1][far, :, 0] = 8.0
    pool[int(bt[1, far // page]), 0, :, far % page, 0] = 8.0
    positions, row_req, qblk = [], [], []
    kernel, bq, tile = ops.attention_plan(group, hd, dtype, decode_only, prefer, page)
    assert kernel == {"generic": "generic", "mma": "mma_keys" if decode_only else "mma_rows", "tcgen05": "tc_rows"}[prefer]
    if kernel == "generic" and split < tile:         # ranges of 32 keys: tiles of 32 (less shared memory than planned)
        tile = split
    r0 = 0
    for r, (c, n) in enumerate(ctx):
        positions += list(range(c, c + n)); row_req += [r] * n
        for b in range(0, n, bq):
            qblk.append((r, r0 + b, min(bq, n - b)))
        r0 += n
    positions_t = torch.tensor(positions, dtype=torch.int32, device=DEV)
    qblk_t = torch.tensor(qblk, dtype=torch.int32, device=DEV)
    out = torch.full((rows, nh * hd), float("nan"), dtype=dtype, device=DEV)
    status = ops.new_status(DEV)
    qd = q.reshape(rows, nh * hd).to(DEV).contiguous()
    scale = 1.0 / math.sqrt(hd)
    ops.attention(qd, qd.stride(0), pool.to(DEV), bt.to(DEV), positions_t, qblk_t, len(qblk), max(positions), rows,
                  nh, nkv, hd, window or 0, split, tile, bq, scale, out, status, kernel)
    ops.raise_on_status(status)
    # reference: every request's rows against its whole key/value sequence
    want = torch.empty(rows, nh * hd, dtype=torch.float64)
    r0 = 0
    for r, (c, n) in enumerate(ctx):
        t = total[r]
        qfull = torch.zeros(t, nh, hd, dtype=torch.float64)
        qfull[c:] = q[r0:r0 + n].double()
        o = plain.attention_fast(qfull, ks[r].double(), vs[r].double(), group, window)
        want[r0:r0 + n] = o[c:]
        r0 += n
    return out.double().cpu(), want


@pytest.mark.parametrize("nh,nkv,hd,page", [(4, 2, 16, 8), (3, 1, 32, 16), (5, 5, 48, 16), (12, 2, 128, 16),
                                            (7, 1, 80, 4), (2, 1, 256, 32), (6, 3, 64, 64)])
def test_attention_float32(ops, nh, nkv, hd, page):
    got, want = _attention_case(ops, nh, nkv, hd, page, torch.float32, None, seed=nh * 100 + hd)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max() < 1e-5 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("nh,nkv,hd,page,window", [(4, 2, 16, 8, 10), (12, 2, 128, 16, 64), (5, 5, 48, 16, 1),
                                                   (3, 1, 32, 16, 100)])
def test_attention_window(ops, nh, nkv, hd, page, window):
    got, want = _attention_case(ops, nh, nkv, hd, page, torch.float32, window, seed=7)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max() < 1e-5 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("nh,nkv,hd,page", [(12, 2, 128, 16), (3, 1, 32, 16), (5, 5, 48, 8)])
def test_attention_bfloat16(ops, nh, nkv, hd, page):
    got, want = _attention_case(ops, nh, nkv, hd, page, torch.bfloat16, None, seed=3)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max() < 1e-2 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("nh,nkv,hd,page,window", [(12, 2, 128, 16, None), (4, 4, 64, 8, None), (14, 2, 64, 32, 40),
                                                   (16, 1, 128, 16, None), (12, 2, 128, 16, 100), (3, 1, 128, 4, None)])
@pytest.mark.parametrize("decode_only", [False, True])
def test_attention_tensor_core_kernel(ops, nh, nkv, hd, page, window, decode_only):
    got, want = _attention_case(ops, nh, nkv, hd, page, torch.bfloat16, window, seed=5, prefer="mma",
                                decode_only=decode_only)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max() < 1e-2 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("nh,nkv,hd,page,window", [(12, 2, 128, 16, None), (4, 4, 64, 8, None), (14, 2, 64, 32, 40),
                                                   (16, 1, 128, 16, None), (12, 2, 128, 16, 100), (3, 1, 128, 4, None),
                                                   (6, 3, 128, 64, None), (8, 2, 64, 1, 50)])
def test_attention_tcgen05_kernel(ops, nh, nkv, hd, page, window):
    got, want = _attention_case(ops, nh, nkv, hd, page, torch.bfloat16, window, seed=5, prefer="tcgen05")
    assert torch.isfinite(got).all()
    assert (got - want).abs().max() < 1e-2 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("prefer,decode_only", [("tcgen05", False), ("mma", False), ("mma", True), ("generic", False)])
@pytest.mark.parametrize("nh,nkv,hd,page,window", [(12, 2, 128, 16, None), (6, 2, 64, 16, 300)])
def test_attention_long_contexts(ops, prefer, decode_only, nh, nkv, hd, page, window):
    got, want = _attention_case(ops, nh, nkv, hd, page, torch.bfloat16, window, seed=9, split=256, prefer=prefer,
                                decode_only=decode_only, long=True)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max() < 1e-2 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("nh,nkv,hd,page,window", [(2, 1, 128, 64, None), (3, 1, 64, 16, None), (2, 2, 128, 32, 700)])
@pytest.mark.parametrize("tile_keys", [128, 64])
def test_attention_tcgen05_long_prompts(ops, nh, nkv, hd, page, window, tile_keys):
    """2,048 rows on top of 6,144 positions of context (8,192 keys), a decoded token at 5,300 and a fresh prompt, in
    one step, in both arrangements of the kernel: tiles of 128 keys, each cut between the two groups of softmax
    warps, and tiles of 64 keys that the groups take in turns (the kernel picks by the number of keys; the test
    moves the limit).  The groups' accumulators are joined at the end.  Against the plain attention."""
    old = ops.attention_wide_from(4096 if tile_keys == 128 else 1 << 30)
    try:
        got, want = _attention_case(ops, nh, nkv, hd, page, torch.bfloat16, window, seed=17, split=256, prefer="tcgen05",
                                    long="wide")
    finally:
        ops.attention_wide_from(old)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max() < 1e-2 * max(1.0, float(want.abs().max()))


def test_attention_refuses_sizes_it_does_not_take(ops):
    with pytest.raises(ops.KernelError, match="head_dim"):
        ops.attention_plan(2, 272)
    with pytest.raises(ops.KernelError, match="tensor-core"):
        ops.attention_plan(2, 48, torch.bfloat16, False, "mma")
    assert ops.attention_plan(2, 48, torch.bfloat16)[0] == "generic"
    assert ops.attention_plan(6, 128, torch.bfloat16, True)[0] == "mma_keys"
    assert ops.attention_plan(32, 128, torch.bfloat16, True)[0] == "generic"      # more than 16 heads per kv head
    assert ops.attention_plan(6, 128, torch.float32)[0] == "generic"


def test_sample_greedy_takes_the_first_maximum(ops):
    V = 1000
    logits = rnd(4, V, seed=11)
    logits[0, 700] = 50.0; logits[0, 300] = 50.0
    logits[1, 999] = 60.0
    logits[2, 0] = 60.0
    logits[3, :] = -1.0
    out = torch.empty(4, dtype=torch.int32, device=DEV)
    ops.sample(logits, None, None, out)
    assert out.tolist() == [300, 999, 0, 0]
    # for a decoding loop on the device: the tokens also go to the step's input buffer, and the positions move on
    # (not for a row that pads the batch); greedy rows and a sampled row alike
    feed = torch.full((4,), -1, dtype=torch.int32, device=DEV)
    positions = torch.tensor([7, 0, 41, 5], dtype=torch.int32, device=DEV)
    advance = torch.tensor([1, 1, 1, 0], dtype=torch.int32, device=DEV)
    temp = torch.tensor([0.0, 0.0, 0.7, 0.0], device=DEV)
    u = torch.tensor([0.0, 0.0, 0.999, 0.0], device=DEV)
    out2 = torch.empty(4, dtype=torch.int32, device=DEV)
    ops.sample(logits, temp, u, out2, feed_tokens=feed, feed_positions=positions, advance=advance)
    assert out2.tolist()[:2] == [300, 999] and out2.tolist()[3] == 0
    assert feed.tolist() == out2.tolist() and positions.tolist() == [8, 1, 42, 5]


def test_sample_temperature_inverts_the_cumulative_distribution(ops):
    V, n = 151, 64
    logits = rnd(n, V, seed=12, scale=2.0)
    temp = torch.full((n,), 0.8, device=DEV)
    temp[5] = 0.0
    u = torch.linspace(0.0, 0.999, n, device=DEV)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    ops.sample(logits, temp, u, out)
    got = out.tolist()
    for r in range(n):
        if r == 5:
            assert got[r] == int(logits[r].argmax())
            continue
        cdf = plain.temperature_cdf(logits[r].cpu(), 0.8)
        lo = 0.0 if got[r] == 0 else float(cdf[got[r] - 1])
        hi = float(cdf[got[r]])
        assert lo - 1e-5 <= float(u[r]) <= hi + 1e-5, (r, got[r], lo, float(u[r]), hi)
    # the same numbers give the same tokens
    out2 = torch.empty(n, dtype=torch.int32, device=DEV)
    ops.sample(logits, temp, u, out2)
    assert out2.tolist() == got
    # a large vocabulary that is no multiple of the block
    V = 151937
    big = rnd(2, V, seed=13)
    t2 = torch.tensor([1.0, 1.0], device=DEV); u2 = torch.tensor([0.25, 0.9], device=DEV)
    o2 = torch.empty(2, dtype=torch.int32, device=DEV)
    ops.sample(big, t2, u2, o2)
    for r in range(2):
        cdf = plain.temperature_cdf(big[r].cpu(), 1.0)
        i = int(o2[r])
        assert (0.0 if i == 0 else float(cdf[i - 1])) - 1e-4 <= float(u2[r]) <= float(cdf[i]) + 1e-4


@pytest.mark.parametrize("T,N,K,splits", [(1, 128, 64, 1), (8, 256, 1536, 1), (8, 2048, 1536, 8), (5, 200, 136, 2),
                                          (16, 1536, 8960, 14), (17, 384, 192, 1), (64, 300, 520, 3),
                                          (100, 256, 256, 1), (300, 520, 328, 1), (2048, 1536, 1536, 1)])
def test_gemm_tcgen05(ops, T, N, K, splits):
    """The tensor-core product against float64, at sizes with ragged edges in all three dimensions."""
    x = rnd(T, K, dtype=torch.bfloat16, seed=21)
    w = rnd(N, K, dtype=torch.bfloat16, seed=22, scale=0.1)
    b = rnd(N, seed=23)
    want = x.double() @ w.double().t() + b.double()
    status = ops.new_status(DEV)
    if splits == 1:
        for dt, tol in ((torch.float32, 2e-5), (torch.bfloat16, 8e-3)):
            out = torch.full((T, N), float("nan"), dtype=dt, device=DEV)
            ops.gemm_bf16_tn(x, w, b, out, 1, status)
            ops.raise_on_status(status)
            assert (out.double() - want).abs().max() <= tol * want.abs().max(), dt
    else:
        out = torch.full((splits, T, N), float("nan"), device=DEV)
        ops.gemm_bf16_tn(x, w, b, out, splits, status)
        ops.raise_on_status(status)
        assert (out.double().sum(0) - want).abs().max() <= 2e-5 * want.abs().max()
    # a row's result does not depend on the rows around it
    if T > 1 and splits == 1:
        one = torch.empty((1, N), device=DEV)
        full = torch.empty((T, N), device=DEV)
        ops.gemm_bf16_tn(x, w, b, full, 1, status)
        ops.gemm_bf16_tn(x[T // 2:T // 2 + 1], w, b, one, 1, status)
        assert torch.equal(one[0], full[T // 2])


def _interleave_gate_up(gate, up):
    """Rows in blocks of 64: gate[0:64], up[0:64], gate[64:128], up[64:128], ..."""
    im = gate.shape[0]
    return torch.stack([gate.reshape(im // 64, 64, -1), up.reshape(im // 64, 64, -1)], 1).reshape(2 * im, -1)


@pytest.mark.gpu
@pytest.mark.parametrize("T,N,K,splits", [(8, 256, 512, 1), (8, 384, 1536, 8), (5, 200, 264, 2), (16, 128, 1024, 4),
                                          (33, 1536, 1536, 8), (64, 300, 640, 2), (17, 256, 192, 1)])
def test_gemm_fused_plain_and_residual(ops, T, N, K, splits):
    torch.manual_seed(T * 31 + N)
    x = (torch.randn(T, K) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.05).to(torch.bfloat16)
    bias = torch.randn(N) * 0.1
    want = x.double() @ w.double().t() + bias.double()
    status = ops.new_status(DEV)
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 1e-2)):
        out = torch.full((T, N), float("nan"), dtype=dtype, device=DEV)
        ops.gemm_fused(w.to(DEV), out, ops.FUSED_PLAIN, x=x.to(DEV), bias=bias.to(DEV), splits=splits, status=status)
        ops.raise_on_status(status)
        assert (out.double().cpu() - want).abs().max() < tol * max(1.0, float(want.abs().max()))
    # residual: the stream is updated in place and the sums of squares of its new rows come back in parts
    stream = torch.randn(T, N)
    xs = stream.clone().to(DEV)
    parts = -(-N // 128) * splits
    ssq = torch.full((parts, 64), float("nan"), device=DEV)
    ops.gemm_fused(w.to(DEV), xs, ops.FUSED_RESIDUAL, x=x.to(DEV), bias=bias.to(DEV), ssq_out=ssq, splits=splits, status=status)
    ops.raise_on_status(status)
    new = stream.double() + want
    assert (xs.double().cpu() - new).abs().max() < 2e-5 * max(1.0, float(new.abs().max()))
    got_ssq = ssq[:, :T].double().sum(0).cpu()
    assert torch.allclose(got_ssq, (xs.double().cpu() ** 2).sum(1), rtol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("T,N,K,splits,parts", [(8, 256, 512, 1, 3), (8, 2048, 1536, 8, 96), (3, 136, 200, 2, 1),
                                               (40, 256, 1536, 4, 12), (64, 128, 640, 1, 5)])
def test_gemm_fused_norm_prologue(ops, T, N, K, splits, parts):
    torch.manual_seed(N + K)
    xf = torch.randn(T, K) * 2.0
    g = (1.0 + 0.2 * torch.randn(K)).to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.05).to(torch.bfloat16)
    eps = 1e-5
    # the sums of squares arrive cut into parts (here: by ranges of columns, as a producing kernel leaves them)
    cols = torch.linspace(0, K, parts + 1).long()
    ssq = torch.zeros(parts, 64)
    for i in range(parts):
        ssq[i, :T] = (xf[:, cols[i]:cols[i + 1]].double() ** 2).sum(1).float()
    rstd = 1.0 / torch.sqrt((xf.double() ** 2).sum(1) / K + eps)
    xn = (xf.double() * rstd[:, None] * g.double()).to(torch.bfloat16)
    want = xn.double() @ w.double().t()
    out = torch.full((T, N), float("nan"), dtype=torch.float32, device=DEV)
    status = ops.new_status(DEV)
    ops.gemm_fused(w.to(DEV), out, ops.FUSED_PLAIN, xf=xf.to(DEV), ssq_in=ssq.to(DEV), norm_weight=g.to(DEV), eps=eps,
                   splits=splits, status=status)
    ops.raise_on_status(status)
    # the operand is rounded to bfloat16 once: a value on a rounding boundary may fall to the other side
    assert (out.double().cpu() - want).abs().max() < 4e-3 * max(1.0, float(want.abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("T,im,K,splits", [(8, 128, 512, 1), (8, 896, 1536, 2), (20, 64, 264, 1), (50, 256, 1024, 8),
                                           (3, 192, 640, 4)])
@pytest.mark.parametrize("bias", [False, True])
def test_gemm_fused_swiglu(ops, T, im, K, splits, bias):
    torch.manual_seed(im + K)
    x = (torch.randn(T, K) * 0.5).to(torch.bfloat16)
    gate = (torch.randn(im, K) * 0.08).to(torch.bfloat16)
    up = (torch.randn(im, K) * 0.08).to(torch.bfloat16)
    bg, bu = (torch.randn(im), torch.randn(im)) if bias else (torch.zeros(im), torch.zeros(im))
    gv, uv = x.double() @ gate.double().t() + bg.double(), x.double() @ up.double().t() + bu.double()
    want = gv / (1.0 + torch.exp(-gv)) * uv
    out = torch.full((T, im), float("nan"), dtype=torch.bfloat16, device=DEV)
    status = ops.new_status(DEV)
    b = _interleave_gate_up(bg[:, None], bu[:, None]).reshape(-1).contiguous().to(DEV) if bias else None
    ops.gemm_fused(_interleave_gate_up(gate, up).contiguous().to(DEV), out, ops.FUSED_SWIGLU, x=x.to(DEV), splits=splits,
                   bias=b, status=status)
    ops.raise_on_status(status)
    assert (out.double().cpu() - want).abs().max() < 1e-2 * max(1.0, float(want.abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("nh,nkv,hd,K,splits", [(12, 2, 128, 1536, 8), (3, 1, 32, 96, 1), (6, 2, 64, 192, 2), (5, 1, 64, 264, 2),
                                                (7, 3, 32, 1024, 16), (1, 1, 128, 128, 1), (28, 4, 128, 512, 2)])
@pytest.mark.parametrize("T", [1, 7, 16, 40])
def test_gemm_fused_rope(ops, nh, nkv, hd, K, splits, T):
    """The q/k/v product with rotation and cache append inside it: tiles that hold whole heads (128), two or four
    heads of different kinds (a query beside a key, a key beside a value), a last tile that is partly empty; the rows
    of three requests at scattered positions, pages in shuffled order, everything not written stays poison; one row
    with a page number outside the pool is reported and writes nothing."""
    torch.manual_seed(nh * 100 + hd + T)
    page, n_pages, max_pages = 16, 23, 6
    N = (nh + 2 * nkv) * hd
    x = (torch.randn(T, K) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.05).to(torch.bfloat16)
    bias = torch.randn(N) * 0.2
    row_req = torch.tensor([t % 3 for t in range(T)], dtype=torch.int32)
    start = [0, 37, 70]
    positions = torch.tensor([start[t % 3] + t // 3 for t in range(T)], dtype=torch.int32)       # request r: start[r], start[r] + 1, ...
    perm = torch.randperm(n_pages)[:3 * max_pages].reshape(3, max_pages).to(torch.int32)
    bt = perm.clone()
    bad_row = T - 1 if T >= 7 else None
    if bad_row is not None:                                            # the last row's page: outside the pool
        positions[bad_row] = 90
        bt[int(row_req[bad_row]), int(positions[bad_row]) // page] = n_pages + 5
        for t in range(T):                                             # (no other row may share that page)
            assert t == bad_row or (int(row_req[t]), int(positions[t]) // page) != (int(row_req[bad_row]), int(positions[bad_row]) // page)
    inv = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -(2 * torch.arange(hd // 2, dtype=torch.float64)) / hd).float().to(DEV)
    table = torch.empty((T, hd // 2, 2), device=DEV)
    ops.rope_table(positions.to(DEV), inv, table)
    pool = torch.full((n_pages, 2, nkv, page, hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    q_out = torch.full((T, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    status = ops.new_status(DEV)
    ops.gemm_fused_rope(w.to(DEV), x.to(DEV), bias.to(DEV), q_out, table, positions.to(DEV), row_req.to(DEV), bt.to(DEV),
                        pool, nh, nkv, hd, splits=splits, status=status)
    torch.cuda.synchronize()
    word = int(status.item())
    assert word == (ops.STATUS_BAD_PAGE if bad_row is not None else 0)
    status.zero_()
    o = (x.double() @ w.double().t() + bias.double()).reshape(T, nh + 2 * nkv, hd)
    c, s_ = table[..., 0].double().cpu()[:, None, :], table[..., 1].double().cpu()[:, None, :]

    def rotate(v):
        a, b = v[..., :hd // 2], v[..., hd // 2:]
        return torch.cat([a * c - b * s_, b * c + a * s_], dim=-1)

    scale = max(1.0, float(o.abs().max()))
    assert (q_out.double().cpu().reshape(T, nh, hd) - rotate(o[:, :nh])).abs().max() < 1e-2 * scale
    k, v = rotate(o[:, nh:nh + nkv]), o[:, nh + nkv:]
    written = 0
    for t in range(T):
        if t == bad_row:
            continue
        pg, sl = int(bt[int(row_req[t]), int(positions[t]) // page]), int(positions[t]) % page
        assert (pool[pg, 0, :, sl].double().cpu() - k[t]).abs().max() < 1e-2 * scale
        assert (pool[pg, 1, :, sl].double().cpu() - v[t]).abs().max() < 1e-2 * scale
        written += 1
    assert int(torch.isfinite(pool.float()).sum()) == written * 2 * nkv * hd       # nothing else was written


@pytest.mark.gpu
@pytest.mark.parametrize("T,N,K,bias", [(256, 256, 64, False), (300, 520, 200, True), (2048, 1536, 1536, True),
                                        (1000, 1288, 456, False), (65, 8, 72, True), (777, 17920 // 8, 1536, False),
                                        (2048, 4096, 128, True), (3000, 2600, 72, False)])
def test_gemm_pair_plain(ops, T, N, K, bias):
    """The product of many rows by pairs of CTAs (tokens on the M side, tiles of 256 tokens x 256, 192 or 128
    features, persistent): sizes that do not fill a tile in any direction, more tiles than pairs, every tile
    width (the last two shapes take 256, (2048, 1536) takes 192, (1000, 1288) takes 128), a bias."""
    torch.manual_seed(T + N)
    x = (torch.randn(T, K) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.05).to(torch.bfloat16)
    b = torch.randn(N) if bias else None
    want = x.double() @ w.double().t() + (b.double() if bias else 0.0)
    out = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    status = ops.new_status(DEV)
    ops.gemm_pair(x.to(DEV), w.to(DEV), out, ops.PAIR_PLAIN, b.to(DEV) if bias else None, status)
    ops.raise_on_status(status)
    assert torch.isfinite(out).all()
    assert (out.double().cpu() - want).abs().max() < 1e-2 * max(1.0, float(want.abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("T,N,K,bias", [(256, 256, 64, False), (300, 520, 200, True), (2048, 1536, 1536, False),
                                        (1000, 1288, 456, True), (65, 8, 72, True), (2048, 4096, 128, True)])
def test_gemm_pair_residual(ops, T, N, K, bias):
    """The same adding into the float residual stream: out += product (+ bias), nothing else of the stream touched."""
    torch.manual_seed(T + N + 1)
    x = (torch.randn(T, K) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.05).to(torch.bfloat16)
    b = torch.randn(N) if bias else None
    stream = torch.randn(T + 3, N)
    want = stream.double().clone()
    want[:T] += x.double() @ w.double().t() + (b.double() if bias else 0.0)
    out = stream.to(DEV)
    status = ops.new_status(DEV)
    ops.gemm_pair(x.to(DEV), w.to(DEV), out[:T], ops.PAIR_RESIDUAL, b.to(DEV) if bias else None, status)
    ops.raise_on_status(status)
    assert (out.double().cpu() - want).abs().max() < 2e-3 * max(1.0, float(want.abs().max()))
    assert torch.equal(out[T:].cpu(), stream[T:])


@pytest.mark.gpu
@pytest.mark.parametrize("T,im,K", [(256, 128, 64), (300, 320, 200), (2048, 8960 // 4, 1536), (999, 64, 136),
                                    (2048, 2048, 72)])
def test_gemm_pair_swiglu(ops, T, im, K):
    """The same with SwiGLU in the epilogue: the weight's rows are gate and up features interleaved in blocks of 64."""
    torch.manual_seed(T + im)
    x = (torch.randn(T, K) * 0.5).to(torch.bfloat16)
    gate = (torch.randn(im, K) * 0.08).to(torch.bfloat16)
    up = (torch.randn(im, K) * 0.08).to(torch.bfloat16)
    g, u = x.double() @ gate.double().t(), x.double() @ up.double().t()
    want = g / (1.0 + torch.exp(-g)) * u
    out = torch.full((T, im), float("nan"), dtype=torch.bfloat16, device=DEV)
    status = ops.new_status(DEV)
    ops.gemm_pair(x.to(DEV), _interleave_gate_up(gate, up).contiguous().to(DEV), out, ops.PAIR_SWIGLU, None, status)
    ops.raise_on_status(status)
    assert torch.isfinite(out).all()
    assert (out.double().cpu() - want).abs().max() < 1e-2 * max(1.0, float(want.abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("nh,nkv,hd,page,dtype,split", [(4, 2, 64, 16, torch.float32, 32), (6, 2, 128, 64, torch.bfloat16, 32),
                                                        (2, 1, 256, 32, torch.float32, 32), (3, 1, 32, 8, torch.float32, 64)])
@pytest.mark.parametrize("decode_only", [False, True])
def test_attention_merge_of_many_ranges(ops, nh, nkv, hd, page, dtype, split, decode_only):
    """Keys cut into far more ranges than the one-trip merge takes (up to 138 of 32 keys): the general merge,
    whose lanes hold the first 128 ranges' maxima and read the rest again."""
    got, want = _attention_case(ops, nh, nkv, hd, page, dtype, None, seed=hd + split, split=split, prefer="generic",
                                decode_only=decode_only, long=True)
    assert torch.isfinite(got).all()
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert (got - want).abs().max() < tol * max(1.0, float(want.abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("nh,nkv,hd,page,window", [(6, 2, 128, 64, 300), (4, 2, 64, 16, 1000), (3, 1, 48, 16, 77)])
@pytest.mark.parametrize("decode_only", [False, True])
def test_attention_merge_of_many_ranges_behind_a_window(ops, nh, nkv, hd, page, window, decode_only):
    """bfloat16 rows over ranges of 32 keys with a window: a row's ranges begin at any number, not at 0, so the
    wide merge's groups of eight ranges are cut at both ends."""
    got, want = _attention_case(ops, nh, nkv, hd, page, torch.bfloat16, window, seed=window, split=32, prefer="generic",
                                decode_only=decode_only, long=True)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max() < 1e-2 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("dtype,page,batch,bound", [(torch.bfloat16, 64, 8, 4095), (torch.bfloat16, 16, 8, 4095),
                                                    (torch.float32, 64, 8, 4095), (torch.bfloat16, 64, 64, 4095),
                                                    (torch.bfloat16, 32, 3, 4095), (torch.bfloat16, 64, 4, 4095),
                                                    (torch.bfloat16, 64, 2, 32767),
                                                    (torch.bfloat16, 64, 1, 20479)])
def test_decoding_attention_under_a_bound_finds_every_needle(ops, dtype, page, batch, bound):
    """Decoding steps that are replayed as a graph launch the attention for the context limit, not for the
    longest request: requests of 40 to 4,000 keys side by side under `max_position` 4095, so that for the short
    ones most CTAs of the fixed grid have nothing to do.  One key of every request is made to win its softmax
    (its value row is a marker), and it is moved through the places where a kernel can lose a key: the first and
    the newest, the two sides of a page's edge and of a 256-key stage, the middle.  Every row must come out as
    its marker; the other keys are noise.  Under a bound of tens of thousands of positions a request's keys are
    spread over dozens of CTAs, whose partial results the wide merge joins; so are the 16 ranges of the three and
    four requests under 4,095 (few rows with more than eight ranges each)."""
    nh, nkv, hd = 12, 2, 128
    lengths = ([40, 700, 1500, 4000, 63, 1023, 255, 2049] * 8)[:batch]
    if batch == 64:
        lengths = [1 + (97 * i) % 4000 for i in range(64)]
    if bound > 4095:
        lengths = [20000, 300][:batch]
    torch.manual_seed(batch + page)
    n_pages_each = [-(-t // page) for t in lengths]
    n_pages = sum(n_pages_each) + 3
    perm = iter(torch.randperm(n_pages).tolist())
    max_pages = (bound + 1) // page
    bt = torch.full((batch, max_pages), -1, dtype=torch.int32)
    pool = torch.full((n_pages, 2, nkv, page, hd), float("nan"), dtype=dtype)
    for r, t in enumerate(lengths):
        k = (torch.randn(t, nkv, hd) * 0.5).to(dtype)
        v = torch.randn(t, nkv, hd).to(dtype)
        for pi in range(n_pages_each[r]):
            pg = next(perm)
            bt[r, pi] = pg
            n = min(page, t - pi * page)
            pool[pg, 0, :, :n] = k[pi * page:pi * page + n].transpose(0, 1)
            pool[pg, 1, :, :n] = v[pi * page:pi * page + n].transpose(0, 1)
    pool = pool.to(DEV)
    q = torch.zeros(batch, nh, hd)
    q[:, :, 5] = 16.0                                   # a needle's score is 16 * 16 / sqrt(128) = 22.6; noise stays under 3
    qd = q.reshape(batch, nh * hd).to(dtype).to(DEV).contiguous()
    positions = torch.tensor([t - 1 for t in lengths], dtype=torch.int32, device=DEV)
    kernel, bq, tile = ops.attention_plan(nh // nkv, hd, dtype, True, "auto", page)
    assert kernel == ("mma_keys" if dtype == torch.bfloat16 else "generic")
    qblk = torch.tensor([(r, r, 1) for r in range(batch)], dtype=torch.int32, device=DEV)
    status = ops.new_status(DEV)
    places = [lambda t: 0, lambda t: t - 1, lambda t: min(t - 1, 63), lambda t: min(t - 1, 64), lambda t: min(t - 1, 255),
              lambda t: min(t - 1, 256), lambda t: t // 2, lambda t: max(0, t - 2), lambda t: (t - 1) // 256 * 256,
              lambda t: max(0, (t - 1) // page * page - 1)]
    for place in places:
        changed = []
        for r, t in enumerate(lengths):
            at = place(t)
            pg, sl = int(bt[r, at // page]), at % page
            changed.append((pg, sl, pool[pg, :, :, sl].clone()))
            pool[pg, 0, :, sl, 5] = 16.0
            pool[pg, 1, :, sl, :] = 100.0 + r
        out = torch.full((batch, nh * hd), float("nan"), dtype=dtype, device=DEV)
        ops.attention(qd, qd.stride(0), pool, bt.to(DEV), positions, qblk, batch, bound, batch, nh, nkv, hd, 0, 256, tile, bq,
                      1.0 / math.sqrt(hd), out, status, kernel)
        ops.raise_on_status(status)
        got = out.float().cpu()
        for r, t in enumerate(lengths):
            assert (got[r] - (100.0 + r)).abs().max() < 1.0, (r, t, place(t), got[r][:4])
        for pg, sl, old in changed:
            pool[pg, :, :, sl] = old
