// Row-wise kernels around the matrix products: embedding gather, residual add fused with RMSNorm,
// SwiGLU, the rotary table of a step, and the rotation of q and k fused with the append of k and v
// to the paged cache.  Statistics, angles and the residual are float; inputs and outputs may be
// float or bfloat16.
#include "common.cuh"

namespace bg {

// ---------------------------------------------------------------------------------------------
// x[t, :] = table[ids[t], :]   (qwen_infer.c:1438-1439).  An id outside the table sets a status
// bit and yields a row of zeros.
template <typename TT>
__global__ void embed_gather_kernel(const TT* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ out, int d, int vocab, unsigned* status) {
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * d;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0 && status) atomicOr(status, BG_STATUS_BAD_TOKEN);
        for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = 0.0f;
        return;
    }
    const TT* row = table + (size_t)id * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = to_float(row[i]);
}

// ---------------------------------------------------------------------------------------------
// For output row r (source row s = rows ? rows[r] : r):
//   v = x[s] (+ delta[s]);  if update: x[s] = v;  out[r] = v * rsqrt(mean(v^2) + eps) * w
// (qwen_infer.c:711-714; the add is the residual sum of :1552 and :1577 moved in front of the norm
// that follows it).  One block per row; the row is held in shared memory between the two passes.
template <typename TD, typename TW, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const TD* __restrict__ delta,
                                   const TW* __restrict__ w, float eps, TO* __restrict__ out,
                                   const int* __restrict__ rows, int d, int update) {
    extern __shared__ float row_buf[];
    __shared__ float red[32];
    const int r = blockIdx.x;
    const int s = rows ? rows[r] : r;
    float* xr = x + (size_t)s * d;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = xr[i];
        if (delta) v += to_float(delta[(size_t)s * d + i]);
        row_buf[i] = v;
        if (update) xr[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    TO* o = out + (size_t)r * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x)
        o[i] = from_float<TO>(row_buf[i] * inv * to_float(w[i]));
}

// x[t] += delta[t] without a norm (the last residual add when no norm follows).
template <typename TD>
__global__ void add_residual_kernel(float* __restrict__ x, const TD* __restrict__ delta, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += to_float(delta[i]);
}

// ---------------------------------------------------------------------------------------------
// out[t, i] = silu(gu[t, i]) * gu[t, im + i]   with silu(g) = g / (1 + exp(-g))  (qwen_infer.c:727-733)
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int rows, int im) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t total = (size_t)rows * im;
    if (idx >= total) return;
    size_t t = idx / im;
    int i = (int)(idx - t * im);
    float g = to_float(gu[t * 2 * (size_t)im + i]);
    float u = to_float(gu[t * 2 * (size_t)im + im + i]);
    out[idx] = from_float<T>((g / (1.0f + expf(-g))) * u);
}

// ---------------------------------------------------------------------------------------------
// cos_sin[t, i] = (cos, sin)(positions[t] * inv_freq[i]), float product of the position converted
// to float, as qwen_infer.c:791-794 computes it once per token for all layers and heads.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float2* __restrict__ cos_sin, int T, int half) {
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= T * half) return;
    int t = idx / half, i = idx - t * half;
    float ang = (float)positions[t] * inv_freq[i];
    float s, c;
    sincosf(ang, &s, &c);
    cos_sin[idx] = make_float2(c, s);
}

// ---------------------------------------------------------------------------------------------
// For token t of request row_req[t] at position positions[t]:
//   rotate every q head in place, and (when kv_pool is given) rotate every k head and store it
//   together with v into the page block_table[req][pos / page_size] at slot pos % page_size.
// Pairs are (i, i + half) for split-half and (2i, 2i + 1) for interleaved pairing
// (qwen_infer.c:782-790); features from rot on are copied.  qkv rows are [q | k | v].
// The pool of one layer is [num_pages][2][nkv][page_size][hd].
template <typename TA, typename TC>
__global__ void rope_kv_append_kernel(TA* __restrict__ qkv, int row_stride, const float2* __restrict__ cos_sin,
                                      const int* __restrict__ positions, const int* __restrict__ row_req,
                                      const int* __restrict__ block_table, int max_pages,
                                      TC* __restrict__ kv_pool, int num_pages, int page_size,
                                      int nh, int nkv, int hd, int rot, int interleaved, unsigned* status) {
    const int t = blockIdx.x;
    const int half = rot >> 1;
    TA* row = qkv + (size_t)t * row_stride;
    const float2* cs = cos_sin ? cos_sin + (size_t)t * half : nullptr;
    // q heads, in place
    if (half > 0) {
        for (int idx = threadIdx.x; idx < nh * half; idx += blockDim.x) {
            int h = idx / half, i = idx - h * half;
            int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
            TA* v = row + (size_t)h * hd;
            float a = to_float(v[ia]), b = to_float(v[ib]);
            float2 f = cs[i];
            v[ia] = from_float<TA>(a * f.x - b * f.y);
            v[ib] = from_float<TA>(b * f.x + a * f.y);
        }
    }
    if (!kv_pool) return;
    const int pos = positions[t];
    const int req = row_req[t];
    const int page = block_table[(size_t)req * max_pages + pos / page_size];
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0 && status) atomicOr(status, BG_STATUS_BAD_PAGE);
        return;
    }
    const int slot = pos % page_size;
    const TA* k = row + (size_t)nh * hd;
    const TA* vv = k + (size_t)nkv * hd;
    TC* kdst = kv_pool + ((size_t)page * 2 + 0) * nkv * page_size * hd;
    TC* vdst = kv_pool + ((size_t)page * 2 + 1) * nkv * page_size * hd;
    for (int idx = threadIdx.x; idx < nkv * hd; idx += blockDim.x) {
        int h = idx / hd, i = idx - h * hd;
        size_t dst = ((size_t)h * page_size + slot) * hd + i;
        vdst[dst] = from_float<TC>(to_float(vv[idx]));
        float val;
        if (i < rot) {
            int pi, partner;
            bool first;
            if (interleaved) { pi = i >> 1; first = (i & 1) == 0; partner = first ? i + 1 : i - 1; }
            else { first = i < half; pi = first ? i : i - half; partner = first ? i + half : i - half; }
            float me = to_float(k[(size_t)h * hd + i]), other = to_float(k[(size_t)h * hd + partner]);
            float2 f = cs[pi];
            val = first ? (me * f.x - other * f.y) : (me * f.x + other * f.y);
        } else {
            val = to_float(k[idx]);
        }
        kdst[dst] = from_float<TC>(val);
    }
}

}  // namespace bg

using namespace bg;

extern "C" int bg_embed_gather(const void* table, int table_dtype, const int* ids, float* out, int T,
                               int d, int vocab, unsigned* status, cudaStream_t stream) {
    if (T <= 0) return BG_OK;
    BG_DISPATCH_DTYPE(table_dtype, TT, embed_gather_kernel<TT><<<T, 256, 0, stream>>>(
        (const TT*)table, ids, out, d, vocab, status));
    BG_LAUNCH_CHECK();
    return BG_OK;
}

template <typename TD, typename TW>
static int add_rmsnorm_out(float* x, const void* delta, const void* w, float eps, void* out, int out_dtype,
                           const int* rows, int n_rows, int d, int update, cudaStream_t stream) {
    size_t smem = (size_t)d * sizeof(float);
    if (smem > 200 * 1024) return BG_ERR_SHAPE;
    if (out_dtype == BG_DTYPE_F32) {
        auto kern = add_rmsnorm_kernel<TD, TW, float>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        kern<<<n_rows, 256, smem, stream>>>(x, (const TD*)delta, (const TW*)w, eps, (float*)out, rows, d, update);
    } else if (out_dtype == BG_DTYPE_BF16) {
        auto kern = add_rmsnorm_kernel<TD, TW, __nv_bfloat16>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        kern<<<n_rows, 256, smem, stream>>>(x, (const TD*)delta, (const TW*)w, eps, (__nv_bfloat16*)out, rows, d, update);
    } else {
        return BG_ERR_DTYPE;
    }
    BG_LAUNCH_CHECK();
    return BG_OK;
}

// delta may be null (then delta_dtype is ignored); rows may be null (then row r reads source row r).
extern "C" int bg_add_rmsnorm(float* x, const void* delta, int delta_dtype, const void* w, int w_dtype,
                              float eps, void* out, int out_dtype, const int* rows, int n_rows, int d,
                              int update, cudaStream_t stream) {
    if (n_rows <= 0) return BG_OK;
    if (!delta) delta_dtype = BG_DTYPE_F32;
    BG_DISPATCH_DTYPE(delta_dtype, TD, BG_DISPATCH_DTYPE(w_dtype, TW,
        return (add_rmsnorm_out<TD, TW>(x, delta, w, eps, out, out_dtype, rows, n_rows, d, update, stream))));
    return BG_OK;
}

extern "C" int bg_add_residual(float* x, const void* delta, int delta_dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return BG_OK;
    unsigned blocks = (unsigned)((n + 255) / 256);
    BG_DISPATCH_DTYPE(delta_dtype, TD, add_residual_kernel<TD><<<blocks, 256, 0, stream>>>(x, (const TD*)delta, (size_t)n));
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_swiglu(const void* gu, void* out, int dtype, int rows, int im, cudaStream_t stream) {
    if (rows <= 0) return BG_OK;
    size_t total = (size_t)rows * im;
    unsigned blocks = (unsigned)((total + 255) / 256);
    BG_DISPATCH_DTYPE(dtype, T, swiglu_kernel<T><<<blocks, 256, 0, stream>>>((const T*)gu, (T*)out, rows, im));
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_rope_table(const int* positions, const float* inv_freq, float* cos_sin, int T, int half,
                             cudaStream_t stream) {
    if (T <= 0 || half <= 0) return BG_OK;
    int total = T * half;
    rope_table_kernel<<<(total + 255) / 256, 256, 0, stream>>>(positions, inv_freq, (float2*)cos_sin, T, half);
    BG_LAUNCH_CHECK();
    return BG_OK;
}

template <typename TA>
static int rope_kv_cache(void* qkv, int row_stride, const float* cos_sin, const int* positions, const int* row_req,
                         const int* block_table, int max_pages, void* kv_pool, int cache_dtype, int num_pages,
                         int page_size, int T, int nh, int nkv, int hd, int rot, int interleaved, unsigned* status,
                         cudaStream_t stream) {
    BG_DISPATCH_DTYPE(cache_dtype, TC, rope_kv_append_kernel<TA, TC><<<T, 256, 0, stream>>>(
        (TA*)qkv, row_stride, (const float2*)cos_sin, positions, row_req, block_table, max_pages,
        (TC*)kv_pool, num_pages, page_size, nh, nkv, hd, rot, interleaved, status));
    BG_LAUNCH_CHECK();
    return BG_OK;
}

// kv_pool may be null: then only q is rotated (a mixer that reads another stage's cache).
extern "C" int bg_rope_kv_append(void* qkv, int act_dtype, int row_stride, const float* cos_sin, const int* positions,
                                 const int* row_req, const int* block_table, int max_pages, void* kv_pool,
                                 int cache_dtype, int num_pages, int page_size, int T, int nh, int nkv, int hd,
                                 int rot, int interleaved, unsigned* status, cudaStream_t stream) {
    if (T <= 0) return BG_OK;
    if (rot < 0 || rot > hd || (rot & 1)) return BG_ERR_SHAPE;
    if (rot > 0 && !cos_sin) return BG_ERR_SHAPE;
    if (!kv_pool) cache_dtype = BG_DTYPE_F32;
    BG_DISPATCH_DTYPE(act_dtype, TA, return (rope_kv_cache<TA>(qkv, row_stride, cos_sin, positions, row_req, block_table,
        max_pages, kv_pool, cache_dtype, num_pages, page_size, T, nh, nkv, hd, rot, interleaved, status, stream)));
    return BG_OK;
}
