// The sampling entry point that allocates nothing: see sample_no_alloc.h for who needs it, what it
// costs and the rules for its caller.
#include "sample_no_alloc.h"

#include <stdio.h>

#include <mutex>

#include "common.cuh"

// The two-stage sampler of sampling.cu, which takes its scratch from the caller.
extern "C" int bg_sample(const float* logits, int n, int V, const float* temperature, const float* uniform, int* out,
                         void* scratch, cudaStream_t stream);
extern "C" long long bg_sample_scratch_bytes(int n);

namespace {

constexpr int kChunks = 64;                     // stage-one blocks per row (SAMPLE_CHUNKS of sampling.cu)
constexpr int kBytesPerRow = kChunks * 12;      // a float maximum, an int index and a float sum per chunk
constexpr int kMaxDevices = 64;

// The scratch itself.  In host code this name is only a handle for cudaGetSymbolAddress; the
// address that kernels can use is looked up below, once per device.
static __device__ __align__(256) unsigned char g_sample_scratch[BG_SAMPLE_NO_ALLOC_MAX_ROWS * kBytesPerRow];

std::mutex g_mu;
void* g_scratch_addr[kMaxDevices] = {nullptr};

int fail(char* err, int err_len, int code, const char* fmt, long long a = 0, long long b = 0) {
    if (err && err_len > 0) snprintf(err, (size_t)err_len, fmt, a, b);
    return code;
}

}  // namespace

extern "C" int bg_sample_no_alloc(const float* logits, int n, int V, const float* temperature, const float* uniform,
                                  int* out, cudaStream_t stream, char* err, int err_len) {
    if (err && err_len > 0) err[0] = '\0';
    if (n <= 0) return BG_OK;
    if (n > BG_SAMPLE_NO_ALLOC_MAX_ROWS)
        return fail(err, err_len, BG_ERR_SHAPE,
                    "bg_sample_no_alloc: %lld rows asked for, but the built-in scratch holds %lld; split the call",
                    n, BG_SAMPLE_NO_ALLOC_MAX_ROWS);
    if (V <= 0 || !logits || !out)
        return fail(err, err_len, BG_ERR_SHAPE, "bg_sample_no_alloc: logits and out must be given and V (%lld) positive", V);
    if (temperature && !uniform)
        return fail(err, err_len, BG_ERR_SHAPE, "bg_sample_no_alloc: temperatures were given without uniform numbers");
    if (bg_sample_scratch_bytes(n) > (long long)sizeof(g_sample_scratch))
        return fail(err, err_len, BG_ERR_SHAPE, "bg_sample_no_alloc: the sampler wants %lld bytes of scratch, the array has %lld",
                    bg_sample_scratch_bytes(n), (long long)sizeof(g_sample_scratch));

    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(err, err_len, (int)e, "bg_sample_no_alloc: cudaGetDevice failed (error %lld)", (long long)e);
    if (dev < 0 || dev >= kMaxDevices)
        return fail(err, err_len, BG_ERR_UNSUPPORTED, "bg_sample_no_alloc: device %lld is beyond the %lld this library tracks", dev, kMaxDevices);
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        if (!g_scratch_addr[dev]) {
            // set-up, once per device, with that device current: the array's address on THIS device
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_sample_scratch);
            if (e != cudaSuccess || !p)
                return fail(err, err_len, e != cudaSuccess ? (int)e : BG_ERR_UNSUPPORTED,
                            "bg_sample_no_alloc: cudaGetSymbolAddress failed on device %lld (error %lld)", dev, (long long)e);
            g_scratch_addr[dev] = p;
        }
        scratch = g_scratch_addr[dev];
    }
    int rc = bg_sample(logits, n, V, temperature, uniform, out, scratch, stream);
    if (rc != BG_OK) return fail(err, err_len, rc, "bg_sample_no_alloc: the sampling kernels could not be launched (code %lld)", rc);
    return BG_OK;
}
