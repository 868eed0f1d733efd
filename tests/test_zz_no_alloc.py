"""The sampling entry point that allocates nothing, called through its exported C symbol.

Some callers of this library cannot allocate device memory when they sample: code running inside a
stream capture, serving loops that must not enter an allocator, and plain-C hosts with a fixed
memory plan.  `bg_sample_no_alloc` keeps the sampler's scratch in a fixed array inside the library.
This test calls it twice in a row, with different inputs, and wants the same tokens as the ordinary
entry point (whose scratch the caller allocates) gives; tokens are integers, so "the same" is exact.
The file sorts last so that a run that stops at the first failure has run everything else before."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
MAX_ROWS = 256


def entry():
    from beglin_b200.csrc import build
    lib = build.load()
    fn = lib.bg_sample_no_alloc
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int]
    fn.restype = ctypes.c_int
    return fn


def call(fn, logits, temperature, uniform, out):
    err = ctypes.create_string_buffer(256)
    rc = fn(logits.data_ptr(), logits.shape[0], logits.shape[1],
            None if temperature is None else temperature.data_ptr(), None if uniform is None else uniform.data_ptr(),
            out.data_ptr(), torch.cuda.current_stream().cuda_stream, err, len(err))
    return rc, err.value.decode()


def test_no_alloc_sampling_matches_the_ordinary_entry_point_twice_in_a_row():
    from beglin_b200.csrc import ops
    fn = entry()
    g = torch.Generator().manual_seed(77)
    for round_, (n, V) in enumerate([(7, 1000), (MAX_ROWS, 3001)]):
        logits = (torch.randn(n, V, generator=g) * 3).to(DEV)
        temperature = torch.full((n,), 0.7, device=DEV)
        temperature[::3] = 0.0                                   # every third row greedy
        uniform = torch.rand(n, generator=g).to(DEV)
        want = torch.empty(n, dtype=torch.int32, device=DEV)
        ops.sample(logits, temperature, uniform, want)
        got = torch.full((n,), -1, dtype=torch.int32, device=DEV)
        before = torch.cuda.memory_allocated()
        rc, msg = call(fn, logits, temperature, uniform, got)
        assert rc == 0, msg
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before           # nothing came from torch's allocator either
        assert torch.equal(got, want), round_
        greedy = torch.full((n,), -1, dtype=torch.int32, device=DEV)
        rc, msg = call(fn, logits, None, None, greedy)
        assert rc == 0, msg
        assert torch.equal(greedy.long(), logits.argmax(dim=1))


def test_no_alloc_sampling_refuses_more_rows_than_its_scratch_holds():
    fn = entry()
    n = MAX_ROWS + 1
    logits = torch.zeros((n, 16), device=DEV)
    out = torch.full((n,), -7, dtype=torch.int32, device=DEV)
    rc, msg = call(fn, logits, None, None, out)
    assert rc != 0 and "256" in msg and "257" in msg
    torch.cuda.synchronize()
    assert int((out != -7).sum()) == 0                           # nothing was launched
    t = torch.ones(4, device=DEV)
    rc, msg = call(fn, logits[:4], t, None, out[:4])
    assert rc != 0 and "uniform" in msg
