"""Python faces of the CUDA kernels: each takes torch tensors on a CUDA device, checks what the
kernel assumes (types, shapes, contiguity), and launches on torch's current stream.

There is no other implementation behind these functions.  If the library cannot be built or
loaded, or a tensor is not on a CUDA device, they raise.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import build as _build

F32, BF16 = 0, 1
STATUS_BAD_TOKEN, STATUS_BAD_PAGE, STATUS_TIMEOUT = 1, 2, 4

_c_int, _c_float, _c_void_p, _c_ll = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong
_c_ull = ctypes.c_ulonglong

_SIGNATURES = {
    "bg_embed_gather": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_float, _c_void_p, _c_void_p],
    "bg_softcap": [_c_void_p, _c_ll, _c_float, _c_void_p],
    "bg_fill_normal": [_c_void_p, _c_int, _c_ll, _c_ull, _c_ll, _c_float, _c_float, _c_void_p],
    "bg_add_rmsnorm": [_c_void_p, _c_void_p, _c_int, _c_int, _c_ll, _c_void_p, _c_int, _c_float, _c_void_p, _c_int,
                       _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
    "bg_add_residual": [_c_void_p, _c_void_p, _c_int, _c_ll, _c_void_p],
    "bg_swiglu": [_c_void_p, _c_int, _c_int, _c_ll, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "bg_rope_table": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p],
    "bg_rope_kv_append": [_c_void_p, _c_int, _c_int, _c_int, _c_ll, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p,
                          _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                          _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "bg_attention_plan": [_c_int, _c_int, ctypes.POINTER(_c_int), ctypes.POINTER(_c_int)],
    "bg_attention_partial": [_c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int,
                             _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
                             _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_void_p, _c_void_p],
    "bg_attention_merge": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int,
                           _c_int, _c_int, _c_int, _c_void_p],
    "bg_attention_mma_plan": [_c_int, _c_int, _c_int, ctypes.POINTER(_c_int)],
    "bg_attention_mma_partial": [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p,
                                 _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                 _c_int, _c_float, _c_void_p, _c_int, _c_void_p, _c_void_p],
    "bg_attention_tc_plan": [_c_int, _c_int, _c_int, ctypes.POINTER(_c_int)],
    "bg_attention_tc": [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int,
                        _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_void_p, _c_void_p],
    "bg_gemm_f32_nt": [_c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
                       _c_int, _c_void_p],
    "bg_gemm_bf16_tn": [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_int,
                        _c_int, _c_int, _c_void_p, _c_void_p],
    "bg_gemm_pair": [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_int,
                     _c_void_p, _c_void_p],
    "bg_gemm_fused": [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_int,
                      _c_void_p, _c_float, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_int,
                      _c_void_p, _c_void_p],
    "bg_gemm_fused_rope": [_c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_int,
                           _c_void_p, _c_float, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p,
                           _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                           _c_void_p],
    "bg_sample": [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "bg_sample_feed": [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                       _c_void_p],
}

_lib = None


class KernelError(RuntimeError):
    pass


def lib():
    global _lib
    if _lib is None:
        handle = _build.load()
        for name, argtypes in _SIGNATURES.items():
            try:
                fn = getattr(handle, name)
            except AttributeError as e:
                raise KernelError(f"the kernel library lacks '{name}'") from e
            fn.argtypes = argtypes
            fn.restype = _c_int
        _lib = handle
    return _lib


def available() -> bool:
    """True when a CUDA device is present.  (The library itself builds without one.)"""
    return torch.cuda.is_available()


_ARG_ERRORS = {-1: "unsupported element type", -2: "unsupported shape", -3: "misaligned tensor",
               -4: "sizes that this kernel does not take"}


_launches = 0


def launch_count() -> int:
    """How many kernels of this library have been launched (or recorded into a graph) so far."""
    return _launches


def count_launches(n: int) -> None:
    """Account for kernels that a replayed CUDA graph launched."""
    global _launches
    _launches += n


def _check(rc: int, name: str) -> None:
    global _launches
    if rc == 0:
        _launches += 1
        return
    if rc < 0:
        raise KernelError(f"{name}: refused: {_ARG_ERRORS.get(rc, rc)}")
    raise KernelError(f"{name}: CUDA error {rc} at launch")


# ------------------------------------------------------------------------------------------------
# Phase timers (the reference's QWEN_PROF, qwen_infer.c:1224-1235): while a profile is open, every kernel
# class is bracketed by two CUDA events on the launching stream; `profile_end` adds up the device time
# between them per class.  Closed, `phase` hands out one shared do-nothing context.
class _NoPhase:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


class _Phase:
    __slots__ = ("name", "start")

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        self.start = torch.cuda.Event(enable_timing=True)
        self.start.record()

    def __exit__(self, *exc):
        end = torch.cuda.Event(enable_timing=True)
        end.record()
        _profile.append((self.name, self.start, end))
        return False


_NO_PHASE = _NoPhase()
_profile = None            # None: closed; a list of (class, start event, end event) while open
_depth = 0


def phase(name: str):
    """Context for the launches of one kernel class.  Phases do not nest: inside an open phase an inner
    one is part of it."""
    if _profile is None:
        return _NO_PHASE
    return _Outer(name)


class _Outer(_Phase):
    def __enter__(self):
        global _depth
        _depth += 1
        if _depth == 1:
            super().__enter__()

    def __exit__(self, *exc):
        global _depth
        if _depth == 1:
            super().__exit__(*exc)
        _depth -= 1
        return False


def profile_begin() -> None:
    global _profile, _depth
    _profile, _depth = [], 0


def profile_end() -> dict:
    """Close the profile: {kernel class: (device milliseconds, brackets)} in order of first use.  Waits for
    the device."""
    global _profile
    records, _profile = _profile or [], None
    torch.cuda.synchronize()
    out = {}
    for name, start, end in records:
        ms, n = out.get(name, (0.0, 0))
        out[name] = (ms + start.elapsed_time(end), n + 1)
    return out


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"tensors must be float32 or bfloat16, got {t.dtype}")


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("beglin_b200 kernels run on a CUDA device only; got a tensor on " + str(t.device))


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The raw handle of torch's current stream on the current device (a cheap call; the public
    torch.cuda.current_stream() costs several microseconds, which counts at hundreds of launches a step)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _i32(t: torch.Tensor, what: str) -> None:
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{what} must be a contiguous int32 tensor")


def new_status(device) -> torch.Tensor:
    return torch.zeros(1, dtype=torch.int32, device=device)


def raise_on_status(status: torch.Tensor) -> None:
    """Read the status word (this waits for the device) and raise if a kernel recorded a fault."""
    v = int(status.item())
    if v == 0:
        return
    status.zero_()
    what = []
    if v & STATUS_BAD_TOKEN:
        what.append("a token id outside the vocabulary")
    if v & STATUS_BAD_PAGE:
        what.append("a block-table entry outside the page pool")
    if v & STATUS_TIMEOUT:
        what.append("a bounded wait inside a kernel ran out")
    raise KernelError("a kernel recorded: " + "; ".join(what or [f"status {v}"]))


# ------------------------------------------------------------------------------------------------
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status: Optional[torch.Tensor],
                 scale: float = 1.0) -> None:
    """out[t] = table[ids[t]] * scale as float32; an id outside the table sets BG_STATUS_BAD_TOKEN."""
    _cuda(table, ids, out)
    _i32(ids, "ids")
    T, d = ids.numel(), table.shape[1]
    if out.dtype != torch.float32 or tuple(out.shape) != (T, d) or not out.is_contiguous() or not table.is_contiguous():
        raise KernelError("embed_gather: out must be contiguous float32 [T, d] and the table contiguous")
    with phase("emb_gather"):
        _check(lib().bg_embed_gather(_p(table), _dt(table), _p(ids), _p(out), T, d, table.shape[0], float(scale), _p(status),
                                     _stream()), "embed_gather")


def fill_normal(out: torch.Tensor, key: int, mean: float, std: float, first: int = 0) -> None:
    """out (contiguous, float32 or bfloat16) = mean + std * x(key, first + i) for its elements i in storage order: the
    counter-based generator of weights/counter_random.py on the device, with the same bits."""
    _cuda(out)
    if not out.is_contiguous():
        raise KernelError("fill_normal: a contiguous tensor")
    _check(lib().bg_fill_normal(_p(out), _dt(out), out.numel(), int(key) & ((1 << 64) - 1), int(first), float(mean), float(std),
                                _stream()), "fill_normal")


def softcap(x: torch.Tensor, cap: float) -> None:
    """x = cap * tanh(x / cap) in place; x contiguous float32 (logits)."""
    _cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous() or not cap > 0.0:
        raise KernelError("softcap: contiguous float32 values and a positive cap")
    _check(lib().bg_softcap(_p(x), x.numel(), float(cap), _stream()), "softcap")


def _parts(t: torch.Tensor, what: str):
    """(number of partial sums, elements between them) of a product's result: [T, N], or
    [parts, T, N] float32 from a split-K product."""
    if t.dim() == 2:
        return 1, 0
    if t.dim() == 3 and t.is_contiguous():
        return t.shape[0], t.shape[1] * t.shape[2]
    raise KernelError(f"{what} must be [T, N] or contiguous [parts, T, N]")


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None, update: bool = True) -> None:
    """v = x[s] (+ delta[s], or the sum over p of delta[p][s]); x[s] = v when update;
    out[r] = rmsnorm(v) * weight, s = rows[r] or r."""
    _cuda(x, delta, weight, out, rows)
    d = x.shape[1]
    n = rows.numel() if rows is not None else x.shape[0]
    if x.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous() or not weight.is_contiguous():
        raise KernelError("add_rmsnorm: x must be contiguous float32; out and weight contiguous")
    if tuple(out.shape) != (n, d) or weight.numel() != d:
        raise KernelError(f"add_rmsnorm: out is {tuple(out.shape)}, expected {(n, d)}; weight has {weight.numel()} of {d}")
    parts, stride = 0, 0
    if delta is not None:
        parts, stride = _parts(delta, "add_rmsnorm: delta")
        if tuple(delta.shape[-2:]) != tuple(x.shape) or not delta.is_contiguous():
            raise KernelError("add_rmsnorm: delta must be contiguous and shaped like x")
    if rows is not None:
        _i32(rows, "rows")
    with phase("rmsnorm"):
        _check(lib().bg_add_rmsnorm(_p(x), _p(delta), _dt(delta) if delta is not None else F32, parts, stride, _p(weight),
                                    _dt(weight), float(eps), _p(out), _dt(out), _p(rows), n, d, 1 if update else 0,
                                    _stream()), "add_rmsnorm")


def add_residual(x: torch.Tensor, delta: torch.Tensor) -> None:
    _cuda(x, delta)
    if x.dtype != torch.float32 or x.shape != delta.shape or not x.is_contiguous() or not delta.is_contiguous():
        raise KernelError("add_residual: x must be contiguous float32 and delta shaped like it")
    with phase("residuals"):
        _check(lib().bg_add_residual(_p(x), _p(delta), _dt(delta), x.numel(), _stream()), "add_residual")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, block: int = 0) -> None:
    """out[t, i] = silu(g[t, i]) * g[t, im + i], g = gate_up or the sum of its partial sums.  With
    `block` > 0 the columns of g are interleaved in blocks of that many: gate, up, gate, up, ..."""
    _cuda(gate_up, out)
    parts, stride = _parts(gate_up, "swiglu: gate_up")
    rows, two_im = gate_up.shape[-2:]
    im = two_im // 2
    if two_im != 2 * im or tuple(out.shape) != (rows, im):
        raise KernelError("swiglu: gate_up must be [rows, 2*im] and out [rows, im]")
    if not gate_up.is_contiguous() or not out.is_contiguous():
        raise KernelError("swiglu: tensors must be contiguous")
    if block < 0 or (block > 0 and im % block):
        raise KernelError(f"swiglu: blocks of {block} do not divide {im} features")
    with phase("swiglu"):
        _check(lib().bg_swiglu(_p(gate_up), _dt(gate_up), parts, stride, _p(out), _dt(out), rows, im, block, _stream()),
               "swiglu")


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = (cos, sin)(positions[t] * inv_freq[i]); out is float32 [T, half, 2]."""
    _cuda(positions, inv_freq, out)
    _i32(positions, "positions")
    T, half = positions.numel(), inv_freq.numel()
    if inv_freq.dtype != torch.float32 or out.dtype != torch.float32 or tuple(out.shape) != (T, half, 2) \
            or not out.is_contiguous() or not inv_freq.is_contiguous():
        raise KernelError("rope_table: inv_freq float32 [half], out contiguous float32 [T, half, 2]")
    with phase("rope"):
        _check(lib().bg_rope_table(_p(positions), _p(inv_freq), _p(out), T, half, _stream()), "rope_table")


def rope_kv_append(src: torch.Tensor, q_out: torch.Tensor, n_rows: int, nh: int, nkv: int, hd: int, rot: int,
                   interleaved: bool, cos_sin: Optional[torch.Tensor], positions: torch.Tensor, row_req: torch.Tensor,
                   block_table: torch.Tensor, kv_pool: Optional[torch.Tensor], page_size: int,
                   status: Optional[torch.Tensor]) -> None:
    """Rows [q | k | v] of `src` ([T, W], or partial sums [parts, T, W]): rotate q into q_out [T, nh*hd],
    rotate k and store k and v into kv_pool [num_pages, 2, nkv, page_size, hd] through the block table
    [B, max_pages].  With kv_pool None the rows hold q only."""
    _cuda(src, q_out, cos_sin, positions, row_req, block_table, kv_pool)
    _i32(positions, "positions"); _i32(row_req, "row_req"); _i32(block_table, "block_table")
    parts, stride = _parts(src, "rope_kv_append: src")
    width = src.shape[-1]
    need = nh * hd + (2 * nkv * hd if kv_pool is not None else 0)
    if src.stride(-1) != 1 or width < need:
        raise KernelError(f"rope_kv_append: rows of {width} features cannot hold q, k, v ({need})")
    if q_out.data_ptr() == src.data_ptr() or q_out.stride(1) != 1 or q_out.shape[1] < nh * hd or q_out.shape[0] < n_rows:
        raise KernelError("rope_kv_append: q_out must be a separate [T, nh*hd] tensor")
    num_pages = 0
    if kv_pool is not None:
        if tuple(kv_pool.shape[1:]) != (2, nkv, page_size, hd) or not kv_pool.is_contiguous():
            raise KernelError(f"rope_kv_append: kv_pool is {tuple(kv_pool.shape)}, expected [pages, 2, {nkv}, {page_size}, {hd}]")
        num_pages = kv_pool.shape[0]
    if rot > 0 and (cos_sin is None or cos_sin.shape[0] < n_rows or cos_sin.shape[1] != rot // 2 or cos_sin.dtype != torch.float32):
        raise KernelError("rope_kv_append: cos_sin must be float32 [T, rot/2, 2]")
    with phase("rope+kv_write"):
        _check(lib().bg_rope_kv_append(_p(src), _dt(src), src.stride(-2), parts, stride, _p(q_out), _dt(q_out),
                                       q_out.stride(0), _p(cos_sin), _p(positions), _p(row_req), _p(block_table),
                                       block_table.shape[1], _p(kv_pool), _dt(kv_pool) if kv_pool is not None else F32,
                                       num_pages, page_size, n_rows, nh, nkv, hd, rot, 1 if interleaved else 0,
                                       _p(status), _stream()), "rope_kv_append")



# choices of `prefer` under which prompt portions run the tcgen05 kernel
def attention_wide_from(keys: int = 0) -> int:
    """The number of keys from which the tcgen05 prompt attention walks tiles of 128 keys instead of 64 (measured
    default 24,576; BEGLIN_B200_ATTN_WIDE_FROM overrides it).  A positive `keys` sets it; the old value is returned."""
    fn = lib().bg_attention_tc_wide_from
    fn.argtypes, fn.restype = [_c_int], _c_int
    return int(fn(int(keys)))


TC_ROWS_FOR = ("auto", "tcgen05")


def attention_plan(group: int, hd: int, dtype: torch.dtype = torch.float32, decode_only: bool = False,
                   prefer: str = "auto", page_size: int = 64) -> Tuple[str, int, int]:
    """(kernel, rows per query block, keys per tile) for these sizes.  Kernels: "mma_keys" (tensor
    cores, one token per block, for steps of single tokens), "mma_rows" (tensor cores, up to 64 rows
    per block) and "generic" (CUDA cores, every size up to head_dim 256, float or bfloat16)."""
    L = lib()
    if prefer not in ("auto", "generic", "mma", "tcgen05"):
        raise KernelError(f"unknown attention kernel choice '{prefer}'")
    if dtype == torch.bfloat16 and not decode_only and prefer in TC_ROWS_FOR:
        bq = _c_int(0)
        if L.bg_attention_tc_plan(group, hd, page_size, ctypes.byref(bq)) == 0:
            return "tc_rows", bq.value, 64
        if prefer == "tcgen05":
            raise KernelError(f"the tcgen05 attention kernel does not take head_dim {hd} with {group} query heads "
                              f"per kv head and pages of {page_size} (head_dim 64 or 128; at most 128 heads per kv head; "
                              "a page size that divides 64)")
    if dtype == torch.bfloat16 and prefer != "generic":
        bq = _c_int(0)
        if L.bg_attention_mma_plan(group, hd, 1 if decode_only else 0, ctypes.byref(bq)) == 0:
            return ("mma_keys" if decode_only else "mma_rows"), bq.value, 64
        if prefer == "mma":
            raise KernelError(f"the tensor-core attention kernel does not take head_dim {hd} with {group} query "
                              "heads per kv head (head_dim 64 or 128; at most 64 heads per kv head)")
    bq, tile = _c_int(0), _c_int(0)
    rc = L.bg_attention_plan(group, hd, ctypes.byref(bq), ctypes.byref(tile))
    if rc != 0:
        raise KernelError(f"attention: head_dim {hd} with {group} query heads per kv head is not supported "
                          "(head_dim must be at most 256)")
    return "generic", bq.value, tile.value


_sm_counts = {}


def sm_count(device=None) -> int:
    """The number of SMs of `device` (default: the current CUDA device), read from the device once."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    if index is None:
        index = torch.cuda.current_device()
    n = _sm_counts.get(index)
    if n is None:
        n = _sm_counts[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return n


def decode_splits(n_streams: int, context: int, sms: Optional[int] = None) -> int:
    """How many CTAs share the keys of one (request, kv head) stream in the decoding kernel.  A CTA has
    a shared-memory buffer per warp and is alone on its SM, so the streams are cut to make one wave
    of CTAs (one per SM; `sms` defaults to the current device's count): more CTAs wait for a second
    wave, fewer leave SMs idle while the others walk longer ranges.  No more than one CTA per 256 keys
    of `context` (a stage of 64 for each of the four warps).  Each request's keys are spread evenly
    over its CTAs by the kernel itself, by the request's own length, so the count depends on the
    shapes of the step only."""
    if sms is None:
        sms = sm_count()
    want = max(1, min(sms // max(1, n_streams), -(-context // 256)))
    per = -(-(-(-context // want)) // 256) * 256          # what the kernel makes of it: whole multiples of 256 keys
    return -(-context // per)                             # no CTA without keys


def attention(*args, **kwargs) -> None:
    """`_attention` under the phase timer of its kernel class (the partial kernel and its merge together)."""
    with phase("attn"):
        _attention(*args, **kwargs)


def _attention(q: torch.Tensor, q_stride: int, kv_pool: torch.Tensor, block_table: torch.Tensor,
              positions: torch.Tensor, qblk: torch.Tensor, n_qblk: int, max_position: int, n_rows: int, nh: int,
              nkv: int, hd: int, window: int, split: int, tile: int, bq: int, scale: float, out: torch.Tensor,
              status: Optional[torch.Tensor], kernel: str = "generic") -> None:
    """Paged grouped-query attention of a step's rows; out is [T, nh*hd].  `kernel`, `bq` and `tile`
    come from `attention_plan`; `qblk` must be cut for that `bq`; `max_position` is the largest
    position among the rows (or a bound on it).

    "generic" cuts the keys into splits of `split` positions (the same boundaries for every request),
    writes partial results and merges them; "mma_keys" (decoding) spreads every request's own keys over
    `decode_splits` CTAs and merges likewise; "mma_rows" and "tc_rows" let one CTA walk all keys of its
    query block and write `out` directly."""
    _cuda(q, kv_pool, block_table, positions, qblk, out)
    _i32(positions, "positions"); _i32(block_table, "block_table")
    if qblk is not None:
        _i32(qblk, "qblk")
    elif kernel != "mma_keys" or n_qblk != n_rows:
        raise KernelError("attention: only the decoding kernel runs without a list of query blocks (block i = row i)")
    if kernel == "tc_rows" and status is None:
        raise KernelError("attention: the tcgen05 kernel wants a status word (its waits are bounded)")
    num_pages, two, nkv_, page_size, hd_ = kv_pool.shape
    if (two, nkv_, hd_) != (2, nkv, hd) or not kv_pool.is_contiguous():
        raise KernelError(f"attention: kv_pool is {tuple(kv_pool.shape)}, expected [pages, 2, {nkv}, page, {hd}]")
    if out.stride(1) != 1 or out.shape[1] < nh * hd or out.shape[0] < n_rows:
        raise KernelError("attention: out must be [T, nh*hd] with unit inner stride")
    L = lib()
    if kernel == "tc_rows":
        if q.dtype != torch.bfloat16 or kv_pool.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
            raise KernelError("attention: the tcgen05 kernel takes bfloat16 queries, caches and outputs")
        _check(L.bg_attention_tc(_p(q), q_stride, _p(kv_pool), num_pages, page_size, _p(block_table),
                                 block_table.shape[1], _p(positions), _p(qblk), n_qblk, _p(out), out.stride(0), nh, nkv,
                                 hd, window, float(scale), int(max_position), _p(status), _stream()), "attention_tcgen05")
        return
    if kernel == "mma_rows":
        if q.dtype != torch.bfloat16 or kv_pool.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
            raise KernelError("attention: the tensor-core kernel takes bfloat16 queries, caches and outputs")
        _check(L.bg_attention_mma_partial(_p(q), q_stride, _p(kv_pool), num_pages, page_size, _p(block_table),
                                          block_table.shape[1], _p(positions), _p(qblk), n_qblk, None, None, 1, 1,
                                          nh, nkv, hd, window, split, 0, float(scale), _p(out), out.stride(0),
                                          _p(status), _stream()), "attention_mma")
        return
    if kernel == "mma_keys":
        split, n_splits = 0, decode_splits(n_qblk * nkv, max_position + 1)
        if n_splits == 1:                        # one CTA walks all keys of its (request, kv head) and writes the rows
            if q.dtype != torch.bfloat16 or kv_pool.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
                raise KernelError("attention: the tensor-core kernel takes bfloat16 queries, caches and outputs")
            _check(L.bg_attention_mma_partial(_p(q), q_stride, _p(kv_pool), num_pages, page_size, _p(block_table),
                                              block_table.shape[1], _p(positions), _p(qblk) if qblk is not None else None,
                                              n_qblk, None, None, 1, 1, nh, nkv, hd, window, 0, 1, float(scale), _p(out),
                                              out.stride(0), _p(status), _stream()), "attention_mma_keys")
            return
    else:
        n_splits = max_position // split + 1
    part_o = torch.empty((n_rows * nh * n_splits, hd), dtype=torch.float32, device=q.device)
    part_ml = torch.empty((n_rows * nh * n_splits, 2), dtype=torch.float32, device=q.device)
    if kernel == "generic":
        _check(L.bg_attention_partial(_p(q), _dt(q), q_stride, _p(kv_pool), _dt(kv_pool), num_pages, page_size,
                                      _p(block_table), block_table.shape[1], _p(positions), _p(qblk), n_qblk,
                                      _p(part_o), _p(part_ml), n_splits, n_splits, nh, nkv, hd, window, split, tile,
                                      bq, float(scale), _p(status), _stream()), "attention_partial")
    elif kernel == "mma_keys":
        if q.dtype != torch.bfloat16 or kv_pool.dtype != torch.bfloat16:
            raise KernelError("attention: the tensor-core kernel takes bfloat16 queries and caches")
        _check(L.bg_attention_mma_partial(_p(q), q_stride, _p(kv_pool), num_pages, page_size, _p(block_table),
                                          block_table.shape[1], _p(positions), _p(qblk) if qblk is not None else None,
                                          n_qblk, _p(part_o),
                                          _p(part_ml), n_splits, n_splits, nh, nkv, hd, window, split, 1,
                                          float(scale), None, 0, _p(status), _stream()), "attention_mma_partial")
    else:
        raise KernelError(f"unknown attention kernel '{kernel}'")
    _check(L.bg_attention_merge(_p(part_o), _p(part_ml), _p(positions), _p(out), _dt(out), out.stride(0), n_rows, nh,
                                hd, n_splits, split, window, _stream()), "attention_merge")


def gemm_f32_nt(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                accumulate: bool = False) -> None:
    """out[M, N] (+)= a[M, K] @ w[N, K]^T (+ bias), all float32, CUDA cores only."""
    _cuda(a, w, bias, out)
    for t in (a, w, out) + ((bias,) if bias is not None else ()):
        if t.dtype != torch.float32:
            raise KernelError("gemm_f32_nt takes float32 tensors")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N or a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError(f"gemm_f32_nt: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not fit")
    if bias is not None and (bias.numel() != N or not bias.is_contiguous()):
        raise KernelError("gemm_f32_nt: bias must have one value per output feature")
    _check(lib().bg_gemm_f32_nt(_p(a), a.stride(0), _p(w), w.stride(0), _p(bias), _p(out), out.stride(0), M, N, K,
                                1 if accumulate else 0, _stream()), "gemm_f32_nt")


def gemm_bf16_tn(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                 splits: int = 1, status: Optional[torch.Tensor] = None) -> None:
    """out = x[T, K] @ w[N, K]^T (+ bias) on the tcgen05 tensor cores, bfloat16 in, float accumulation.
    `out` is [T, N] (float32 or bfloat16) for splits == 1, or float32 [splits, T, N] partial sums over
    ranges of K, which the consumer adds up in index order (the bias is in partial 0)."""
    _cuda(x, w, bias, out, status)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_bf16_tn takes bfloat16 operands")
    T, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or x.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError(f"gemm_bf16_tn: shapes x{tuple(x.shape)} w{tuple(w.shape)} do not fit")
    if K % 8 or x.stride(0) % 8 or w.stride(0) % 8:
        raise KernelError("gemm_bf16_tn: the inner size and the row strides must be multiples of 8 (TMA wants "
                          "16-byte row strides)")
    want = (T, N) if splits == 1 else (splits, T, N)
    if tuple(out.shape) != want or not out.is_contiguous():
        raise KernelError(f"gemm_bf16_tn: out is {tuple(out.shape)}, expected contiguous {want}")
    if splits > 1 and out.dtype != torch.float32:
        raise KernelError("gemm_bf16_tn: partial sums are float32")
    if splits > (K + 63) // 64:
        raise KernelError("gemm_bf16_tn: more splits than 64-wide blocks of K")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N or not bias.is_contiguous()):
        raise KernelError("gemm_bf16_tn: bias must be float32 with one value per output feature")
    _check(lib().bg_gemm_bf16_tn(_p(w), N, K, w.stride(0), _p(x), T, x.stride(0), _p(bias), _p(out), _dt(out), N,
                                 splits, _p(status), _stream()), "gemm_bf16_tn")


def gemm_bf16_tn_unchecked(x: torch.Tensor, w_ptr: int, n_out: int, k: int, ldw: int, bias_ptr, out: torch.Tensor,
                           splits: int, status_ptr) -> None:
    """gemm_bf16_tn for a caller that has checked the weight once (Linear): x must be contiguous
    bfloat16 [T, k] and out contiguous [T, n_out] or float32 [splits, T, n_out]."""
    _check(_lib.bg_gemm_bf16_tn(w_ptr, n_out, k, ldw, x.data_ptr(), x.shape[0], x.stride(0), bias_ptr, out.data_ptr(),
                                F32 if out.dtype == torch.float32 else BF16, n_out, splits, status_ptr, _stream()),
           "gemm_bf16_tn")


PAIR_PLAIN, PAIR_SWIGLU, PAIR_RESIDUAL = 0, 1, 2


def gemm_pair(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int = PAIR_PLAIN,
              bias: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None) -> None:
    """The product of many rows (prompt portions) with w[N, K]^T by pairs of CTAs on the tcgen05 tensor cores.
    mode PAIR_PLAIN: out bfloat16 [T, N] = product (+ bias).  mode PAIR_SWIGLU: w's rows are interleaved (64 of
    gate, then their 64 of up); out bfloat16 [T, N / 2] = silu(gate) * up.  mode PAIR_RESIDUAL: out is the float32
    residual stream [T, N]: out += product (+ bias)."""
    _cuda(x, w, out, bias, status)
    N, K = w.shape
    T = x.shape[0]
    cols = N // 2 if mode == PAIR_SWIGLU else N
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or \
            out.dtype != (torch.float32 if mode == PAIR_RESIDUAL else torch.bfloat16):
        raise KernelError("gemm_pair takes bfloat16 operands and gives a bfloat16 result (adds to a float32 stream)")
    if x.shape[1] != K or x.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1 or tuple(out.shape) != (T, cols):
        raise KernelError(f"gemm_pair: shapes x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
    if status is None:
        raise KernelError("gemm_pair wants a status word (its waits are bounded)")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N or not bias.is_contiguous()):
        raise KernelError("gemm_pair: bias must be float32 with one value per output feature")
    _check(lib().bg_gemm_pair(_p(w), N, K, w.stride(0), _p(x), T, x.stride(0), _p(bias), _p(out), out.stride(0), mode,
                              _p(status), _stream()), "gemm_pair")


def gemm_pair_unchecked(x: torch.Tensor, w_ptr: int, n_out: int, k: int, ldw: int, out: torch.Tensor, mode: int,
                        status_ptr, bias_ptr=None) -> None:
    """gemm_pair for a caller that has checked the weight once (Linear): x bfloat16 [T, k] with contiguous rows,
    out bfloat16 [T, n_out], with PAIR_SWIGLU [T, n_out / 2], with PAIR_RESIDUAL the float32 stream [T, n_out]."""
    if status_ptr is None:
        raise KernelError("gemm_pair wants a status word (its waits are bounded)")
    _check(_lib.bg_gemm_pair(w_ptr, n_out, k, ldw, x.data_ptr(), x.shape[0], x.stride(0), bias_ptr, out.data_ptr(),
                             out.stride(0), mode, status_ptr, _stream()), "gemm_pair")


FUSED_PLAIN, FUSED_RESIDUAL, FUSED_SWIGLU = 0, 1, 2


def gemm_fused(w: torch.Tensor, out: torch.Tensor, mode: int = FUSED_PLAIN, *, x: Optional[torch.Tensor] = None,
               xf: Optional[torch.Tensor] = None, ssq_in: Optional[torch.Tensor] = None,
               norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0, bias: Optional[torch.Tensor] = None,
               ssq_out: Optional[torch.Tensor] = None, splits: int = 1, status: Optional[torch.Tensor] = None) -> None:
    """The product of up to 64 rows with w[N, K]^T on the tcgen05 tensor cores, with its neighbours fused in.

    Left operand: `x` (bfloat16 [T, K]), or the float32 residual stream `xf` [T, K] normalised on the fly:
    bf16(xf * rstd * norm_weight), rstd = 1 / sqrt(sum_p ssq_in[p] / K + eps), ssq_in float32 [parts, >= T].
    K is cut into `splits` (1, 2, 4, 8 or 16) ranges whose CTAs add up inside a thread block cluster.
    mode FUSED_PLAIN: out[T, N] = product (+ bias), float32 or bfloat16.
    mode FUSED_RESIDUAL: out (float32 [T, N], the residual stream) += product (+ bias); ssq_out
      [ceil(N / 128) * splits, >= T] receives partial sums of squares of the new rows.
    mode FUSED_SWIGLU: w's rows are interleaved (64 of gate, then their 64 of up); out bfloat16 [T, N / 2] =
      silu(gate) * up."""
    _cuda(w, out, x, xf, ssq_in, norm_weight, bias, ssq_out, status)
    N, K = w.shape
    if w.dtype != torch.bfloat16 or w.stride(1) != 1:
        raise KernelError("gemm_fused takes a bfloat16 weight with contiguous rows")
    if (x is None) == (xf is None):
        raise KernelError("gemm_fused takes either x (bfloat16) or xf (float32 with ssq_in and norm_weight)")
    src = x if x is not None else xf
    T = src.shape[0]
    if src.shape[1] != K or src.stride(1) != 1 or T > 64:
        raise KernelError(f"gemm_fused: the left operand is {tuple(src.shape)}, expected up to 64 rows of {K}")
    if x is not None and x.dtype != torch.bfloat16:
        raise KernelError("gemm_fused: x must be bfloat16")
    if xf is not None:
        if xf.dtype != torch.float32 or ssq_in is None or norm_weight is None:
            raise KernelError("gemm_fused: xf must be float32 and come with ssq_in and norm_weight")
        if ssq_in.dtype != torch.float32 or ssq_in.dim() != 2 or ssq_in.shape[1] < T or ssq_in.stride(1) != 1:
            raise KernelError("gemm_fused: ssq_in must be float32 [parts, >= T]")
        if norm_weight.dtype != torch.bfloat16 or norm_weight.numel() != K or not norm_weight.is_contiguous():
            raise KernelError("gemm_fused: norm_weight must be bfloat16 with one value per input feature")
    n_cols = N // 2 if mode == FUSED_SWIGLU else N
    if out.shape[0] != T or out.shape[1] != n_cols or out.stride(1) != 1:
        raise KernelError(f"gemm_fused: out is {tuple(out.shape)}, expected {(T, n_cols)}")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N or not bias.is_contiguous()):
        raise KernelError("gemm_fused: bias must be float32 with one value per output feature")
    if mode == FUSED_RESIDUAL and ssq_out is not None:
        parts = -(-N // 128) * splits
        if ssq_out.dtype != torch.float32 or ssq_out.dim() != 2 or ssq_out.shape[0] < parts or ssq_out.shape[1] < T \
                or ssq_out.stride(1) != 1:
            raise KernelError(f"gemm_fused: ssq_out must be float32 [>= {parts}, >= {T}]")
    _check(lib().bg_gemm_fused(_p(w), N, K, w.stride(0), _p(x), x.stride(0) if x is not None else 0, _p(xf),
                               xf.stride(0) if xf is not None else 0, _p(ssq_in),
                               ssq_in.shape[0] if ssq_in is not None else 0, ssq_in.stride(0) if ssq_in is not None else 0,
                               _p(norm_weight), float(eps), T, _p(bias), mode, _p(out), _dt(out), out.stride(0),
                               _p(ssq_out), ssq_out.stride(0) if ssq_out is not None else 0, splits, _p(status),
                               _stream()), "gemm_fused")


def gemm_fused_unchecked(w_ptr: int, n_out: int, k: int, ldw: int, T: int, out: torch.Tensor, mode: int, x, xf, ssq_in,
                         norm_w_ptr, eps: float, bias_ptr, ssq_out, splits: int, status_ptr) -> None:
    """gemm_fused for a caller that has checked the shapes once (Linear)."""
    _check(_lib.bg_gemm_fused(w_ptr, n_out, k, ldw, None if x is None else x.data_ptr(), 0 if x is None else x.stride(0),
                              None if xf is None else xf.data_ptr(), 0 if xf is None else xf.stride(0),
                              None if ssq_in is None else ssq_in.data_ptr(), 0 if ssq_in is None else ssq_in.shape[0],
                              0 if ssq_in is None else ssq_in.stride(0), norm_w_ptr, eps, T, bias_ptr, mode, out.data_ptr(),
                              F32 if out.dtype == torch.float32 else BF16, out.stride(0),
                              None if ssq_out is None else ssq_out.data_ptr(), 0 if ssq_out is None else ssq_out.stride(0),
                              splits, status_ptr, _stream()), "gemm_fused")


def gemm_fused_rope(w: torch.Tensor, x: Optional[torch.Tensor], bias: Optional[torch.Tensor], q_out: torch.Tensor,
                    cos_sin: torch.Tensor, positions: torch.Tensor, row_req: torch.Tensor, block_table: torch.Tensor,
                    kv_pool: torch.Tensor, nh: int, nkv: int, hd: int, splits: int = 1,
                    status: Optional[torch.Tensor] = None, *, xf: Optional[torch.Tensor] = None,
                    ssq_in: Optional[torch.Tensor] = None, norm_weight: Optional[torch.Tensor] = None,
                    eps: float = 0.0) -> None:
    """x [T, K] (bfloat16, up to 64 rows; or the float32 stream xf with ssq_in, norm_weight and eps, as gemm_fused)
    times w [(nh + 2 nkv) hd, K]^T (+ bias), rows [q | k | v]: queries and keys rotated by cos_sin [T, hd / 2, 2]
    (feature d with d + hd / 2), queries to q_out [T, nh hd], keys and values into kv_pool
    [pages, 2, nkv, page_size, hd] at positions[t] of request row_req[t].  hd is 32, 64 or 128."""
    _cuda(w, x, xf, ssq_in, norm_weight, bias, q_out, cos_sin, positions, row_req, block_table, kv_pool, status)
    N, K = w.shape
    if (x is None) == (xf is None):
        raise KernelError("gemm_fused_rope takes either x (bfloat16) or xf (float32 with ssq_in and norm_weight)")
    src = x if x is not None else xf
    T = src.shape[0]
    if w.dtype != torch.bfloat16 or q_out.dtype != torch.bfloat16 or kv_pool.dtype != torch.bfloat16:
        raise KernelError("gemm_fused_rope takes bfloat16 weights, queries and cache")
    if x is not None and x.dtype != torch.bfloat16:
        raise KernelError("gemm_fused_rope: x must be bfloat16")
    if xf is not None:
        if xf.dtype != torch.float32 or ssq_in is None or norm_weight is None:
            raise KernelError("gemm_fused_rope: xf must be float32 and come with ssq_in and norm_weight")
        if ssq_in.dtype != torch.float32 or ssq_in.dim() != 2 or ssq_in.shape[1] < T or ssq_in.stride(1) != 1:
            raise KernelError("gemm_fused_rope: ssq_in must be float32 [parts, >= T]")
        if norm_weight.dtype != torch.bfloat16 or norm_weight.numel() != K or not norm_weight.is_contiguous():
            raise KernelError("gemm_fused_rope: norm_weight must be bfloat16 with one value per input feature")
    if N != (nh + 2 * nkv) * hd or src.shape[1] != K or w.stride(1) != 1 or src.stride(1) != 1 or T > 64:
        raise KernelError(f"gemm_fused_rope: w {tuple(w.shape)}, rows {tuple(src.shape)} for {nh}/{nkv} heads of {hd}")
    if q_out.shape[0] < T or q_out.shape[1] < nh * hd or q_out.stride(1) != 1:
        raise KernelError(f"gemm_fused_rope: q_out is {tuple(q_out.shape)}")
    if kv_pool.dim() != 5 or tuple(kv_pool.shape[1:3]) != (2, nkv) or kv_pool.shape[4] != hd or not kv_pool.is_contiguous():
        raise KernelError(f"gemm_fused_rope: the pool is {tuple(kv_pool.shape)}")
    if cos_sin.dtype != torch.float32 or tuple(cos_sin.shape) != (T, hd // 2, 2) or not cos_sin.is_contiguous():
        raise KernelError(f"gemm_fused_rope: cos_sin is {tuple(cos_sin.shape)}, expected {(T, hd // 2, 2)} float32")
    for t in (positions, row_req, block_table):
        _i32(t, "positions, row_req and block_table")
    if positions.numel() != T or row_req.numel() != T or block_table.dim() != 2 or not block_table.is_contiguous():
        raise KernelError("gemm_fused_rope: positions and row_req have one value per row, block_table is [requests, pages]")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N or not bias.is_contiguous()):
        raise KernelError("gemm_fused_rope: bias must be float32 with one value per output feature")
    gemm_fused_rope_unchecked(w.data_ptr(), K, w.stride(0), T, q_out, x, xf, ssq_in,
                              None if norm_weight is None else norm_weight.data_ptr(), float(eps),
                              None if bias is None else bias.data_ptr(), cos_sin, positions, row_req, block_table, kv_pool,
                              kv_pool.shape[3], nh, nkv, hd, splits, None if status is None else status.data_ptr())


def gemm_fused_rope_unchecked(w_ptr: int, k: int, ldw: int, T: int, q_out: torch.Tensor, x, xf, ssq_in, norm_w_ptr,
                              eps: float, bias_ptr, cos_sin: torch.Tensor, positions: torch.Tensor, row_req: torch.Tensor,
                              block_table: torch.Tensor, kv_pool: torch.Tensor, page_size: int, nh: int, nkv: int, hd: int,
                              splits: int, status_ptr) -> None:
    """The q/k/v product of up to 64 rows with rotation and cache append behind it (left operand as gemm_fused):
    q_out bfloat16 [T, nh hd] receives the rotated queries, kv_pool [pages, 2, nkv, page_size, hd] (bfloat16) the
    rotated keys and the values at each row's position.  For a caller that has checked the shapes (Attention);
    head sizes other than 32, 64 and 128 raise."""
    _check(_lib.bg_gemm_fused_rope(w_ptr, k, ldw, None if x is None else x.data_ptr(), 0 if x is None else x.stride(0),
                                   None if xf is None else xf.data_ptr(), 0 if xf is None else xf.stride(0),
                                   None if ssq_in is None else ssq_in.data_ptr(), 0 if ssq_in is None else ssq_in.shape[0],
                                   0 if ssq_in is None else ssq_in.stride(0), norm_w_ptr, eps, T, bias_ptr,
                                   q_out.data_ptr(), q_out.stride(0), cos_sin.data_ptr(), positions.data_ptr(),
                                   row_req.data_ptr(), block_table.data_ptr(), block_table.shape[1], kv_pool.data_ptr(),
                                   kv_pool.shape[0], page_size, nh, nkv, hd, splits, status_ptr, _stream()),
           "gemm_fused_rope")


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor], uniform: Optional[torch.Tensor],
           out: torch.Tensor, feed_tokens: Optional[torch.Tensor] = None, feed_positions: Optional[torch.Tensor] = None,
           advance: Optional[torch.Tensor] = None) -> None:
    """out[r] = first argmax of logits[r] when temperature[r] <= 0 (or temperature is None), else the
    index where the cumulative softmax(logits[r] / temperature[r]) first exceeds uniform[r].  For a decoding
    step that is replayed on the device: the token also goes to feed_tokens[r] (the step's input buffer), and
    feed_positions[r] grows by advance[r] (by 1 without `advance`)."""
    _cuda(logits, temperature, uniform, out, feed_tokens, feed_positions, advance)
    for t in (feed_tokens, feed_positions, advance):
        if t is not None:
            _i32(t, "feed_tokens, feed_positions and advance")
            if t.numel() != logits.shape[0]:
                raise KernelError("sample: feed_tokens, feed_positions and advance have one value per row")
    n, V = logits.shape
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise KernelError("sample: logits must be contiguous float32 [n, V]")
    _i32(out, "out")
    for t in (temperature, uniform):
        if t is not None and (t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous()):
            raise KernelError("sample: temperature and uniform must be float32 [n]")
    scratch = torch.empty(n * 64 * 3, dtype=torch.float32, device=logits.device)
    with phase("sample"):
        _check(lib().bg_sample_feed(_p(logits), n, V, _p(temperature), _p(uniform), _p(out), _p(scratch), _p(feed_tokens),
                                    _p(feed_positions), _p(advance), _stream()), "sample")
    global _launches
    _launches += 1            # two kernels
