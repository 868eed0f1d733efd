// bg_sample_no_alloc: token sampling for callers that cannot allocate device memory.
//
// This entry point has no counterpart in popixoxipop-collab/beglin (its only sampler is a one-line
// argmax over a host array, qwen_infer.c:2152-2155); it exists for the way this library is used on
// a GPU.
//
// Who needs it.  bg_sample works in two stages and wants a few KB of device scratch per row between
// them, which its caller has to provide, and providing it means a cudaMalloc or a framework's
// allocator.  Some callers may not do that at the moment they sample: code that runs while a CUDA
// stream is being captured into a graph (an allocation there is an error or changes the graph), a
// serving loop whose latency budget has no room for an allocator call that may fall through to the
// driver and synchronise the device, and hosts that link this library from plain C with a fixed
// memory plan, where every byte on the device is accounted for at start-up and nothing may be
// allocated afterwards.  For them the scratch lives inside the library, in a fixed device array.
//
// What it costs.  The array holds BG_SAMPLE_NO_ALLOC_MAX_ROWS rows' worth of scratch,
// 256 rows x 64 chunks x 12 bytes = 196,608 bytes, on every GPU that loads the library, from load
// until the process exits.  A call with more rows is refused (nothing is launched).
//
// Rules for the caller.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress, once
//     per device, with that device current).  That look-up is not a stream operation: make the first
//     call on each device before any stream capture begins.
//   * All calls share the one array, and it keeps what the last call left in it.  Nothing in it has
//     to start at zero: stage one writes every entry that stage two reads, so no clearing is done or
//     needed.  But two calls that overlap on the GPU (different streams, or one stream captured twice
//     and replayed concurrently) write the same entries and race; order them on one stream or with
//     events.
//   * The call itself allocates nothing, on the host or on the device, and calls no routine that
//     does: no cudaMalloc, cudaFree, cudaMallocAsync, and no framework allocator.  Inputs and outputs
//     are the caller's.
#pragma once

#include <cuda_runtime.h>

#define BG_SAMPLE_NO_ALLOC_MAX_ROWS 256

#ifdef __cplusplus
extern "C" {
#endif

// out[r] = index of the first maximum of logits[r, 0..V) when temperature is null or
// temperature[r] <= 0, else the index at which the cumulative softmax(logits[r] / temperature[r])
// first exceeds uniform[r] (uniform in [0, 1), required when temperature is given).
// logits: device float [n, V] contiguous; temperature, uniform: device float [n] or null;
// out: device int [n].  Runs on `stream`.
// Returns 0 on success.  On refusal returns a negative code (or a positive cudaError_t) and, when
// err is not null, writes a message of at most err_len - 1 characters there.
int bg_sample_no_alloc(const float* logits, int n, int V, const float* temperature, const float* uniform,
                       int* out, cudaStream_t stream, char* err, int err_len);

#ifdef __cplusplus
}
#endif
