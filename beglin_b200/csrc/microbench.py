"""Small stand-alone workloads of single kernels, for timing and for profiler captures.

    python -m beglin_b200.csrc.microbench gemm --tokens 8 --out 17920 --inner 1536 --splits 2
    python -m beglin_b200.csrc.microbench gemm-fused --tokens 8 --out 17920 --inner 1536 --splits 2 --norm --mode swiglu
    python -m beglin_b200.csrc.microbench gemm-fused --tokens 8 --inner 1536 --splits 8 --norm --mode rope --heads 12 --kv-heads 2
    python -m beglin_b200.csrc.microbench gemm-pair --tokens 2048 --out 17920 --inner 1536 --mode swiglu [--library]
    python -m beglin_b200.csrc.microbench attention-decode --batch 8 --context 4096
    python -m beglin_b200.csrc.microbench attention-prefill --tokens 2048
    python -m beglin_b200.csrc.microbench norm --tokens 8 --width 1536 --parts 12

Each workload builds inputs larger than the L2 cache where the kernel's traffic is the point (weights
and caches are rotated between launches), launches the kernel a few times inside a CUDA graph, and
prints the time per launch on the device with the bytes or flops per second that it stands for.
"""
from __future__ import annotations

import argparse
import math

import torch

from . import ops

DEV = "cuda:0"


def _time(fn, launches: int) -> float:
    """Microseconds per launch: `fn(i)` recorded `launches` times into a CUDA graph, replayed once warm."""
    for i in range(2):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(launches):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    g.replay()
    t1.record()
    torch.cuda.synchronize()
    return t0.elapsed_time(t1) / launches * 1e3


def gemm(a) -> None:
    T, N, K, S = a.tokens, a.out, a.inner, a.splits
    copies = max(2, min(48, int(300e6 // (N * K * 2)) + 1))
    ws = [(torch.randn(N, K, device=DEV) * 0.02).to(torch.bfloat16) for _ in range(copies)]
    x = torch.randn(T, K, device=DEV).to(torch.bfloat16)
    status = ops.new_status(DEV)
    out = torch.empty((S, T, N) if S > 1 else (T, N), dtype=torch.float32 if S > 1 else torch.bfloat16, device=DEV)
    if a.library:
        us = _time(lambda i: torch.mm(x, ws[i % copies].t()), a.launches)
    else:
        us = _time(lambda i: ops.gemm_bf16_tn(x, ws[i % copies], None, out, S, status), a.launches)
        ops.raise_on_status(status)
    gb = N * K * 2 / 1e9
    print(f"gemm tokens={T} out={N} inner={K} splits={S} {'library' if a.library else 'tcgen05'}: {us:.1f} us  "
          f"{gb / us * 1e6:.0f} GB/s of weights  {2.0 * T * N * K / us / 1e6:.1f} TFLOP/s")


def gemm_fused(a) -> None:
    """The fused few-token product: --norm makes the operand from a float residual stream (RMSNorm inside),
    --mode plain | residual | swiglu | rope picks the epilogue."""
    T, N, K, S = a.tokens, a.out, a.inner, a.splits
    if a.mode == "rope":
        return gemm_fused_rope(a)
    mode = {"plain": ops.FUSED_PLAIN, "residual": ops.FUSED_RESIDUAL, "swiglu": ops.FUSED_SWIGLU}[a.mode]
    copies = max(2, min(48, int(300e6 // (N * K * 2)) + 1))
    ws = [(torch.randn(N, K, device=DEV) * 0.02).to(torch.bfloat16) for _ in range(copies)]
    x = torch.randn(T, K, device=DEV).to(torch.bfloat16)
    xf = torch.randn(T, K, device=DEV)
    g = torch.ones(K, device=DEV, dtype=torch.bfloat16)
    ssq_in = (xf * xf).sum(1)[None, :].repeat(12, 1) / 12
    ssq_in = torch.nn.functional.pad(ssq_in, (0, 64 - T)).contiguous()
    n_cols = N // 2 if mode == ops.FUSED_SWIGLU else N
    out = torch.zeros((T, n_cols), dtype=torch.bfloat16 if mode == ops.FUSED_SWIGLU else torch.float32, device=DEV)
    ssq_out = torch.empty((-(-N // 128) * S, 64), device=DEV) if mode == ops.FUSED_RESIDUAL else None
    status = ops.new_status(DEV)
    kw = dict(xf=xf, ssq_in=ssq_in, norm_weight=g, eps=1e-6) if a.norm else dict(x=x)
    us = _time(lambda i: ops.gemm_fused(ws[i % copies], out, mode, splits=S, ssq_out=ssq_out, status=status, **kw), a.launches)
    ops.raise_on_status(status)
    print(f"gemm-fused tokens={T} out={N} inner={K} splits={S} {'norm -> ' if a.norm else ''}{a.mode}: {us:.1f} us  "
          f"{N * K * 2 / us / 1e3:.0f} GB/s of weights")


def gemm_fused_rope(a) -> None:
    """The q/k/v product of a decoding step with rotation and cache append behind it: --tokens requests at position
    --context - 1, --heads / --kv-heads of --head-dim (the weight has (heads + 2 kv heads) head_dim rows)."""
    T, K, S, nh, nkv, hd, page = a.tokens, a.inner, a.splits, a.heads, a.kv_heads, a.head_dim, 64
    N = (nh + 2 * nkv) * hd
    copies = max(2, min(48, int(300e6 // (N * K * 2)) + 1))
    ws = [(torch.randn(N, K, device=DEV) * 0.02).to(torch.bfloat16) for _ in range(copies)]
    x = torch.randn(T, K, device=DEV).to(torch.bfloat16)
    xf = torch.randn(T, K, device=DEV)
    g = torch.ones(K, device=DEV, dtype=torch.bfloat16)
    ssq_in = (xf * xf).sum(1)[None, :].repeat(12, 1) / 12
    ssq_in = torch.nn.functional.pad(ssq_in, (0, 64 - T)).contiguous()
    bias = torch.randn(N, device=DEV) * 0.1
    pool, bt = _filled_cache(T, a.context, nkv, hd, page)
    positions = torch.full((T,), a.context - 1, dtype=torch.int32, device=DEV)
    row_req = torch.arange(T, dtype=torch.int32, device=DEV)
    inv = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -(2 * torch.arange(hd // 2, dtype=torch.float64)) / hd).float().to(DEV)
    table = torch.empty((T, hd // 2, 2), device=DEV)
    ops.rope_table(positions, inv, table)
    q_out = torch.empty((T, nh * hd), dtype=torch.bfloat16, device=DEV)
    status = ops.new_status(DEV)
    kw = dict(xf=xf, ssq_in=ssq_in, norm_weight=g, eps=1e-6) if a.norm else {}
    us = _time(lambda i: ops.gemm_fused_rope(ws[i % copies], None if a.norm else x, bias, q_out, table, positions, row_req, bt,
                                             pool, nh, nkv, hd, splits=S, status=status, **kw), a.launches)
    ops.raise_on_status(status)
    print(f"gemm-fused tokens={T} heads={nh}/{nkv} head_dim={hd} inner={K} splits={S} {'norm -> ' if a.norm else ''}rope: "
          f"{us:.1f} us  {N * K * 2 / us / 1e3:.0f} GB/s of weights")


def _filled_cache(batch: int, context: int, nkv: int, hd: int, page: int):
    pages_per = -(-context // page)
    n_pages = batch * pages_per
    pool = (torch.randn(n_pages, 2, nkv, page, hd, device=DEV) * 0.5).to(torch.bfloat16)
    perm = torch.randperm(n_pages)
    bt = perm.reshape(batch, pages_per).to(torch.int32).to(DEV).contiguous()
    return pool, bt


def gemm_pair(a) -> None:
    T, N, K = a.tokens, a.out, a.inner
    copies = max(2, min(48, int(300e6 // (N * K * 2)) + 1))
    ws = [(torch.randn(N, K, device=DEV) * 0.02).to(torch.bfloat16) for _ in range(copies)]
    x = torch.randn(T, K, device=DEV).to(torch.bfloat16)
    status = ops.new_status(DEV)
    swiglu, residual = a.mode == "swiglu", a.mode == "residual"
    out = torch.zeros((T, N // 2 if swiglu else N), dtype=torch.float32 if residual else torch.bfloat16, device=DEV)
    if a.library:
        # the library's product; with its neighbour as a kernel of its own (SwiGLU, or the residual add with the norm)
        tmp = torch.empty((T, N), dtype=torch.bfloat16, device=DEV)
        nw = torch.ones(N, dtype=torch.bfloat16, device=DEV)
        normed = torch.empty((T, N), dtype=torch.bfloat16, device=DEV)
        def fn(i):
            torch.mm(x, ws[i % copies].t(), out=tmp)
            if swiglu:
                ops.swiglu(tmp, out, 64)
            elif residual:
                ops.add_rmsnorm(out, tmp, nw, 1e-6, normed)
    else:
        mode = ops.PAIR_SWIGLU if swiglu else ops.PAIR_RESIDUAL if residual else ops.PAIR_PLAIN
        nw = torch.ones(N, dtype=torch.bfloat16, device=DEV)
        normed = torch.empty((T, N), dtype=torch.bfloat16, device=DEV)
        def fn(i):
            ops.gemm_pair(x, ws[i % copies], out, mode, None, status)
            if residual:
                ops.add_rmsnorm(out, None, nw, 1e-6, normed, update=False)
    us = _time(fn, a.launches)
    ops.raise_on_status(status)
    print(f"gemm-pair {'library' if a.library else 'pairs'} mode={a.mode} tokens={T} out={N} inner={K}: {us:.1f} us  "
          f"{2.0 * T * N * K / us / 1e6:.1f} TFLOP/s")


def attention_decode(a) -> None:
    B, ctx, nh, nkv, hd, page = a.batch, a.context, a.heads, a.kv_heads, a.head_dim, a.page
    one = B * ctx * 2 * nkv * hd * 2
    copies = max(1, min(16, int(400e6 // one)))                  # rotate caches so that they come from HBM
    caches = [_filled_cache(B, ctx, nkv, hd, page) for _ in range(copies)]
    kernel, bq, tile = ops.attention_plan(nh // nkv, hd, torch.bfloat16, True, page_size=page)
    q = torch.randn(B, nh * hd, device=DEV).to(torch.bfloat16)
    positions = torch.full((B,), ctx - 1, dtype=torch.int32, device=DEV)
    qblk = torch.stack([torch.arange(B), torch.arange(B), torch.ones(B, dtype=torch.long)], 1).to(torch.int32).to(DEV)
    out = torch.empty((B, nh * hd), dtype=torch.bfloat16, device=DEV)
    status = ops.new_status(DEV)
    us = _time(lambda i: ops.attention(q, q.stride(0), caches[i % copies][0], caches[i % copies][1], positions, qblk, B,
                                       ctx - 1, B, nh, nkv, hd, 0, a.split, tile, bq, 1.0 / math.sqrt(hd), out, status,
                                       kernel), a.launches)
    ops.raise_on_status(status)
    gb = B * ctx * 2 * nkv * hd * 2 / 1e9
    print(f"attention-decode ({kernel}) batch={B} context={ctx} heads={nh}/{nkv} head_dim={hd}: {us:.1f} us  "
          f"{gb / us * 1e6:.0f} GB/s of cache (attention + merge)")


def attention_prefill(a) -> None:
    T, nh, nkv, hd, page = a.tokens, a.heads, a.kv_heads, a.head_dim, a.page
    pool, bt = _filled_cache(1, T, nkv, hd, page)
    kernel, bq, tile = ops.attention_plan(nh // nkv, hd, torch.bfloat16, False, a.kernel, page)
    q = torch.randn(T, nh * hd, device=DEV).to(torch.bfloat16)
    positions = torch.arange(T, dtype=torch.int32, device=DEV)
    blocks = [(0, b, min(bq, T - b)) for b in range(0, T, bq)]
    qblk = torch.tensor(blocks, dtype=torch.int32, device=DEV)
    out = torch.empty((T, nh * hd), dtype=torch.bfloat16, device=DEV)
    status = ops.new_status(DEV)
    us = _time(lambda i: ops.attention(q, q.stride(0), pool, bt, positions, qblk, len(blocks), T - 1, T, nh, nkv, hd,
                                       0, a.split, tile, bq, 1.0 / math.sqrt(hd), out, status, kernel), a.launches)
    ops.raise_on_status(status)
    flops = 4.0 * nh * hd * T * (T + 1) / 2
    print(f"attention-prefill ({kernel}) tokens={T} heads={nh}/{nkv} head_dim={hd}: {us:.1f} us  {flops / us / 1e6:.1f} TFLOP/s")


def norm(a) -> None:
    T, d, parts = a.tokens, a.width, a.parts
    x = torch.randn(T, d, device=DEV)
    delta = torch.randn((parts, T, d) if parts > 1 else (T, d), device=DEV)
    if a.bf16_addend:
        delta = delta.to(torch.bfloat16)
    w = torch.ones(d, dtype=torch.bfloat16, device=DEV)
    out = torch.empty((T, d), dtype=torch.bfloat16, device=DEV)
    us = _time(lambda i: ops.add_rmsnorm(x, delta, w, 1e-6, out), a.launches)
    print(f"norm tokens={T} width={d} parts={parts}: {us:.1f} us")


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="what", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--tokens", type=int, default=8); g.add_argument("--out", type=int, default=17920)
    g.add_argument("--inner", type=int, default=1536); g.add_argument("--splits", type=int, default=1)
    g.add_argument("--library", action="store_true"); g.set_defaults(fn=gemm)
    gp = sub.add_parser("gemm-pair")
    gp.add_argument("--tokens", type=int, default=2048); gp.add_argument("--out", type=int, default=17920)
    gp.add_argument("--inner", type=int, default=1536); gp.add_argument("--mode", default="plain", choices=["plain", "swiglu", "residual"])
    gp.add_argument("--library", action="store_true"); gp.set_defaults(fn=gemm_pair)
    f = sub.add_parser("gemm-fused")
    f.add_argument("--tokens", type=int, default=8); f.add_argument("--out", type=int, default=17920)
    f.add_argument("--inner", type=int, default=1536); f.add_argument("--splits", type=int, default=2)
    f.add_argument("--norm", action="store_true"); f.add_argument("--mode", default="plain", choices=["plain", "residual", "swiglu", "rope"])
    f.add_argument("--heads", type=int, default=12); f.add_argument("--kv-heads", type=int, default=2)
    f.add_argument("--head-dim", type=int, default=128); f.add_argument("--context", type=int, default=4096)
    f.set_defaults(fn=gemm_fused)
    d = sub.add_parser("attention-decode")
    d.add_argument("--batch", type=int, default=8); d.add_argument("--context", type=int, default=4096)
    d.set_defaults(fn=attention_decode)
    p = sub.add_parser("attention-prefill")
    p.add_argument("--tokens", type=int, default=2048); p.set_defaults(fn=attention_prefill)
    p.add_argument("--kernel", default="auto", choices=["auto", "mma", "tcgen05", "generic"])
    for s in (d, p):
        s.add_argument("--heads", type=int, default=12); s.add_argument("--kv-heads", type=int, default=2)
        s.add_argument("--head-dim", type=int, default=128); s.add_argument("--page", type=int, default=64)
        s.add_argument("--split", type=int, default=256)
    n = sub.add_parser("norm")
    n.add_argument("--tokens", type=int, default=8); n.add_argument("--width", type=int, default=1536)
    n.add_argument("--parts", type=int, default=1); n.add_argument("--bf16-addend", action="store_true")
    n.set_defaults(fn=norm)
    for s in (g, gp, f, d, p, n):
        s.add_argument("--launches", type=int, default=20)
    a = ap.parse_args()
    ops.lib()
    a.fn(a)


if __name__ == "__main__":
    main()
