// Row-wise kernels around the matrix products: embedding gather, residual add fused with RMSNorm,
// SwiGLU, the rotary table of a step, and the rotation of q and k fused with the append of k and v
// to the paged cache.  Statistics, angles and the residual are float; inputs and outputs may be
// float or bfloat16.
#include <type_traits>

#include "common.cuh"

namespace bg {

// ---------------------------------------------------------------------------------------------
// x[t, :] = table[ids[t], :] * scale   (qwen_infer.c:1438-1439, where the scale is 1).  An id outside the
// table sets a status bit and yields a row of zeros.
template <typename TT>
__global__ void embed_gather_kernel(const TT* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ out, int d, int vocab, float scale, unsigned* status) {
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * d;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0 && status) atomicOr(status, BG_STATUS_BAD_TOKEN);
        for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = 0.0f;
        return;
    }
    const TT* row = table + (size_t)id * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = to_float(row[i]) * scale;
}

// Random weights on the device: out[i] = mean + std * x(key, first + i), x approximately normal, a function of the
// key and the element's number alone, of integer operations and two exactly rounded float operations, so that the
// host's numpy code (weights/counter_random.py) makes the same bits:
//   h_j = mix64(key + (3 i + j) * GOLDEN), j = 0..2 (splitmix64's finalizer);
//   x = (the sum of the twelve 16-bit fields of h_0..h_2 - 6 * 65535) / 65536.
__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
template <typename TO>
__global__ void fill_normal_kernel(TO* __restrict__ out, long long n, unsigned long long key, long long first, float mean, float std) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const unsigned long long e = (unsigned long long)(first + i);
    int total = 0;
#pragma unroll
    for (int j = 0; j < 3; ++j) {
        const unsigned long long h = mix64(key + (e * 3ull + (unsigned long long)j) * 0x9E3779B97F4A7C15ull);
        total += (int)(h & 0xFFFF) + (int)((h >> 16) & 0xFFFF) + (int)((h >> 32) & 0xFFFF) + (int)(h >> 48);
    }
    const float x = __fmul_rn((float)(total - 6 * 65535), 1.0f / 65536.0f);
    out[i] = from_float<TO>(__fadd_rn(mean, __fmul_rn(std, x)));
}

// x = cap * tanh(x / cap): a cap on the logits of architectures that have one.
__global__ void softcap_kernel(float* __restrict__ x, long long n, float cap) {
    pdl_launch();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

// ---------------------------------------------------------------------------------------------
// For output row r (source row s = rows ? rows[r] : r):
//   v = x[s] + sum_p delta[p][s];  if update: x[s] = v;  out[r] = v * rsqrt(mean(v^2) + eps) * w
// (qwen_infer.c:711-714; the add is the residual sum of :1552 and :1577 moved in front of the norm
// that follows it).  delta may be the partial sums of a split-K product, [parts][T][d], added in
// index order.  One block per row; the row is held in shared memory between the two passes.
template <typename TD, typename TW, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const TD* __restrict__ delta, int parts, size_t part_stride,
                                   const TW* __restrict__ w, float eps, TO* __restrict__ out,
                                   const int* __restrict__ rows, int d, int update) {
    extern __shared__ float row_buf[];
    __shared__ float red[32];
    pdl_launch();
    pdl_wait();
    const int r = blockIdx.x;
    const int s = rows ? rows[r] : r;
    float* xr = x + (size_t)s * d;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = xr[i];
        if (delta) v += sum_parts(delta + (size_t)s * d + i, parts, part_stride);
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

// The same for a width that is a multiple of 8 and 16-byte aligned rows: every thread moves eight
// features with 16-byte loads and stores, so a row of a few thousand features is one round trip.
template <typename TD, typename TW, typename TO>
__global__ void add_rmsnorm_vec8_kernel(float* __restrict__ x, const TD* __restrict__ delta, int parts,
                                        size_t part_stride, const TW* __restrict__ w, float eps, TO* __restrict__ out,
                                        const int* __restrict__ rows, int d, int update) {
    extern __shared__ float row_buf[];
    __shared__ float red[32];
    pdl_launch();
    pdl_wait();
    const int r = blockIdx.x;
    const int s = rows ? rows[r] : r;
    float* xr = x + (size_t)s * d;
    const int d8 = d >> 3;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < d8; c += blockDim.x) {
        float v[8];
        load8(xr + 8 * c, v);
        if (delta) {
            const TD* dp = delta + (size_t)s * d + 8 * c;
            if (std::is_same<TD, float>::value) {
                const float4* d4 = reinterpret_cast<const float4*>(dp);
                float4 a = sum_parts4(d4, parts, part_stride >> 2), b = sum_parts4(d4 + 1, parts, part_stride >> 2);
                v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w; v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
            } else {
                for (int p = 0; p < parts; ++p) {
                    float a[8];
                    load8(dp + (size_t)p * part_stride, a);
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[i] += a[i];
                }
            }
        }
        store8(row_buf + 8 * c, v);
        if (update) store8(xr + 8 * c, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    TO* o = out + (size_t)r * d;
    for (int c = threadIdx.x; c < d8; c += blockDim.x) {
        float v[8], g[8];
        load8(row_buf + 8 * c, v);
        load8(w + 8 * c, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = v[i] * inv * g[i];
        store8(o + 8 * c, v);
    }
}

// The same with a WARP per row and the row in registers (ITER chunks of eight features per lane): all loads of a
// row are on their way at once, the statistics need shuffles only, and no thread waits at a barrier of the block.
// A row's sum of squares is added up in an order that the width alone fixes, whatever the step's other rows are.
template <typename TD, typename TW, typename TO, int ITER>
__global__ void __launch_bounds__(256) add_rmsnorm_warp_kernel(float* __restrict__ x, const TD* __restrict__ delta,
                                                               const TW* __restrict__ w, float eps, TO* __restrict__ out,
                                                               const int* __restrict__ rows, int n_rows, int d, int update) {
    pdl_launch();
    pdl_wait();
    const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (r >= n_rows) return;
    const int s = rows ? rows[r] : r;
    float* xr = x + (size_t)s * d;
    const int d8 = d >> 3;
    float v[ITER][8];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < ITER; ++i) {
        const int c = lane + 32 * i;
        if (c < d8) {
            load8(xr + 8 * c, v[i]);
            if (delta) {
                float a[8];
                load8(delta + (size_t)s * d + 8 * c, a);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[i][j] += a[j];
            }
        }
    }
#pragma unroll
    for (int i = 0; i < ITER; ++i) {
        const int c = lane + 32 * i;
        if (c < d8) {
            if (update && delta) store8(xr + 8 * c, v[i]);
#pragma unroll
            for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
        }
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    TO* o = out + (size_t)r * d;
#pragma unroll
    for (int i = 0; i < ITER; ++i) {
        const int c = lane + 32 * i;
        if (c < d8) {
            float g[8];
            load8(w + 8 * c, g);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[i][j] = v[i][j] * inv * g[j];
            store8(o + 8 * c, v[i]);
        }
    }
}

// For float partial sums and few rows: one float4 per thread, so the loads of all parts of a row are
// in flight at once across the block (the kernel is a chain of dependent round trips otherwise).
template <typename TW, typename TO>
__global__ void __launch_bounds__(512) add_rmsnorm_parts_kernel(float* __restrict__ x, const float* __restrict__ delta, int parts,
                                         size_t part_stride, const TW* __restrict__ w, float eps, TO* __restrict__ out,
                                         const int* __restrict__ rows, int d, int update) {
    extern __shared__ float row_buf[];
    __shared__ float red[32];
    pdl_launch();
    // the norm's weight is written by no kernel of the step: the first chunk's values are fetched while
    // the kernel that produces the addends may still be running
    const int d4 = d >> 2;
    float w0[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if ((int)threadIdx.x < d4) {
#pragma unroll
        for (int j = 0; j < 4; ++j) w0[j] = to_float(w[4 * threadIdx.x + j]);
    }
    pdl_wait();
    const int r = blockIdx.x;
    const int s = rows ? rows[r] : r;
    float4* xr = reinterpret_cast<float4*>(x + (size_t)s * d);
    float4* rb = reinterpret_cast<float4*>(row_buf);
    float ss = 0.0f;
    float4 mine = make_float4(0.0f, 0.0f, 0.0f, 0.0f);          // this thread's first chunk stays in registers
#pragma unroll 1
    for (int i = threadIdx.x; i < d4; i += blockDim.x) {
        float4 a = sum_parts4(reinterpret_cast<const float4*>(delta + (size_t)s * d) + i, parts, part_stride >> 2);
        float4 v = xr[i];
        v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
        if (i == (int)threadIdx.x) mine = v; else rb[i] = v;
        if (update) xr[i] = v;
        ss += v.x * v.x; ss += v.y * v.y; ss += v.z * v.z; ss += v.w * v.w;
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    TO* o = out + (size_t)r * d;
#pragma unroll 1
    for (int i = threadIdx.x; i < d4; i += blockDim.x) {
        const bool first = i == (int)threadIdx.x;
        float4 v = first ? mine : rb[i];
        const float g0 = first ? w0[0] : to_float(w[4 * i + 0]), g1 = first ? w0[1] : to_float(w[4 * i + 1]);
        const float g2 = first ? w0[2] : to_float(w[4 * i + 2]), g3 = first ? w0[3] : to_float(w[4 * i + 3]);
        o[4 * i + 0] = from_float<TO>(v.x * inv * g0);
        o[4 * i + 1] = from_float<TO>(v.y * inv * g1);
        o[4 * i + 2] = from_float<TO>(v.z * inv * g2);
        o[4 * i + 3] = from_float<TO>(v.w * inv * g3);
    }
}

// The same for FEW rows of a bfloat16 step (17 to 64 decoded tokens): a cluster of C CTAs per row, each with a C-th of
// the row's chunks, one float4 per thread.  A block per row leaves the partial sums of 32 rows to 32 SMs (7.2 us for
// rows of 3,584 with 5 parts); the cluster spreads them over C times as many.  The ranks exchange their sums of
// squares through distributed shared memory and add them in rank order: another order than the kernel above uses, so
// this one serves bfloat16 results only (the float path keeps one order for every number of rows).
template <typename TW, typename TO, int C>
__global__ void __launch_bounds__(256) add_rmsnorm_parts_cluster_kernel(float* __restrict__ x, const float* __restrict__ delta,
                                                                        int parts, size_t part_stride, const TW* __restrict__ w,
                                                                        float eps, TO* __restrict__ out, const int* __restrict__ rows,
                                                                        int d, int update) {
    __shared__ float red[32];
    __shared__ float ssq_of[C];                                  // rank c's sum of squares, stored here by rank c
    pdl_launch();
    const int rank = blockIdx.z;                                 // the cluster is (1, 1, C)
    const int d4 = d >> 2, per = (d4 + C - 1) / C;
    const int i = rank * per + (int)threadIdx.x;                 // this thread's chunk of the row
    const bool live = (int)threadIdx.x < per && i < d4;
    float w0[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (live) {                                                  // (the norm's weight is written by no kernel of the step)
#pragma unroll
        for (int j = 0; j < 4; ++j) w0[j] = to_float(w[4 * i + j]);
    }
    cluster_arrive_relaxed();                                    // first use of the barrier: the peers are running
    pdl_wait();
    const int r = blockIdx.x;
    const int s = rows ? rows[r] : r;
    float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float ss = 0.0f;
    if (live) {
        const float4 a = sum_parts4(reinterpret_cast<const float4*>(delta + (size_t)s * d) + i, parts, part_stride >> 2);
        float4* xr = reinterpret_cast<float4*>(x + (size_t)s * d);
        v = xr[i];
        v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
        if (update) xr[i] = v;
        ss += v.x * v.x; ss += v.y * v.y; ss += v.z * v.z; ss += v.w * v.w;
    }
    ss = block_sum(ss, red);
    cluster_wait();
    if ((int)threadIdx.x < C)
        st_cluster(peer_addr((unsigned)__cvta_generic_to_shared(&ssq_of[rank]), threadIdx.x), ss);
    cluster_sync_all();                                          // second use: every rank's sum has arrived everywhere
    float total = 0.0f;
#pragma unroll
    for (int c = 0; c < C; ++c) total += ssq_of[c];
    const float inv = 1.0f / sqrtf(total / (float)d + eps);
    if (live) {
        TO* o = out + (size_t)r * d + 4 * i;
        o[0] = from_float<TO>(v.x * inv * w0[0]);
        o[1] = from_float<TO>(v.y * inv * w0[1]);
        o[2] = from_float<TO>(v.z * inv * w0[2]);
        o[3] = from_float<TO>(v.w * inv * w0[3]);
    }
}

// x[t] += delta[t] without a norm (the last residual add when no norm follows).
template <typename TD>
__global__ void add_residual_kernel(float* __restrict__ x, const TD* __restrict__ delta, size_t n) {
    pdl_launch();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += to_float(delta[i]);
}

// ---------------------------------------------------------------------------------------------
// out[t, i] = silu(g) * u with g = sum_p gu[p][t, i], u = sum_p gu[p][t, im + i] and
// silu(g) = g / (1 + exp(-g))  (qwen_infer.c:727-733).  gu may be the partial sums of a split-K
// product, [parts][rows][2 im].  With block > 0 the columns of gu are interleaved in blocks of that
// many features, gate then up, gate then up (the layout that lets one CTA of the fused product hold
// both): gate i is column (i / block) * 2 block + i % block and its up lies `block` columns on.
// silu(g) * u.  For a bfloat16 result (8 bits of mantissa) the exponential and the reciprocal are the hardware's
// approximations (ex2.approx and the approximate division: relative error about 2^-21), which makes the kernel bound by memory
// instead of by these two functions; a float result is computed with expf and a division.
template <typename TO> __device__ __forceinline__ float silu_mul(float g, float u);
template <> __device__ __forceinline__ float silu_mul<float>(float g, float u) { return (g / (1.0f + expf(-g))) * u; }
template <> __device__ __forceinline__ float silu_mul<__nv_bfloat16>(float g, float u) {
    return __fdividef(g, 1.0f + __expf(-g)) * u;
}

template <typename TI, typename TO>
__global__ void swiglu_kernel(const TI* __restrict__ gu, int parts, size_t part_stride, TO* __restrict__ out,
                              int rows, int im, int block) {
    pdl_launch();
    // where this thread's values lie is integer arithmetic (divisions) on the grid alone: done before the wait
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t total = (size_t)rows * im;
    const bool idle = idx >= total;
    size_t t = idle ? 0 : idx / im;
    int i = idle ? 0 : (int)(idx - t * im);
    const int col = block > 0 ? (i / block) * 2 * block + i % block : i;
    const TI* gp = gu + t * 2 * (size_t)im + col;
    pdl_wait();
    if (idle) return;
    float g = sum_parts(gp, parts, part_stride);
    float u = sum_parts(gp + (block > 0 ? block : im), parts, part_stride);
    out[idx] = from_float<TO>(silu_mul<TO>(g, u));
}

// Float partial sums, im and block multiples of 4: four features per thread, 16-byte loads, the parts added in
// index order as above.
template <typename TO>
__global__ void swiglu_parts_vec4_kernel(const float* __restrict__ gu, int parts, size_t part_stride, TO* __restrict__ out,
                                         int rows, int im, int block) {
    pdl_launch();
    const int im4 = im >> 2;
    const unsigned idx = blockIdx.x * blockDim.x + threadIdx.x;          // (the launcher keeps rows * im / 4 under 2^32)
    const bool idle = idx >= (unsigned)rows * (unsigned)im4;
    const unsigned t = idle ? 0u : idx / (unsigned)im4;
    const int i = idle ? 0 : 4 * (int)(idx - t * (unsigned)im4);
    const int col = block > 0 ? (i / block) * 2 * block + i % block : i;
    const float4* gp = reinterpret_cast<const float4*>(gu + (size_t)t * 2 * (size_t)im + col);
    pdl_wait();
    if (idle) return;
    const float4 g = sum_parts4(gp, parts, part_stride / 4);
    const float4 u = sum_parts4(gp + (block > 0 ? block : im) / 4, parts, part_stride / 4);
    const float r[4] = {silu_mul<TO>(g.x, u.x), silu_mul<TO>(g.y, u.y), silu_mul<TO>(g.z, u.z), silu_mul<TO>(g.w, u.w)};
    TO* o = out + (size_t)t * (size_t)im + i;
    if constexpr (std::is_same<TO, float>::value) {
        *reinterpret_cast<float4*>(o) = make_float4(r[0], r[1], r[2], r[3]);
    } else {
        uint2 raw;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
        h[0] = __floats2bfloat162_rn(r[0], r[1]);
        h[1] = __floats2bfloat162_rn(r[2], r[3]);
        *reinterpret_cast<uint2*>(o) = raw;
    }
}

// One tensor (no partial sums), im a multiple of 8: eight features per thread, 16-byte accesses.
template <typename TI, typename TO>
__global__ void swiglu_vec8_kernel(const TI* __restrict__ gu, TO* __restrict__ out, int rows, int im, int block) {
    pdl_launch();
    const int im8 = im >> 3;
    const unsigned idx = blockIdx.x * blockDim.x + threadIdx.x;          // (the launcher keeps rows * im / 8 under 2^32)
    const bool idle = idx >= (unsigned)rows * (unsigned)im8;
    const size_t t = idle ? 0u : idx / (unsigned)im8;
    const int c = idle ? 0 : (int)(idx - (unsigned)t * (unsigned)im8);
    const int i = 8 * c;                                     // block is a multiple of 8 here
    const int col = block > 0 ? (i / block) * 2 * block + i % block : i;
    pdl_wait();
    if (idle) return;
    float g[8], u[8];
    load8(gu + t * 2 * (size_t)im + col, g);
    load8(gu + t * 2 * (size_t)im + col + (block > 0 ? block : im), u);
#pragma unroll
    for (int i = 0; i < 8; ++i) g[i] = silu_mul<TO>(g[i], u[i]);
    store8(out + t * (size_t)im + 8 * c, g);
}

// ---------------------------------------------------------------------------------------------
// cos_sin[t, i] = (cos, sin)(positions[t] * inv_freq[i]), float product of the position converted
// to float, as qwen_infer.c:791-794 computes it once per token for all layers and heads.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float2* __restrict__ cos_sin, int T, int half) {
    pdl_launch();
    pdl_wait();
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= T * half) return;
    int t = idx / half, i = idx - t * half;
    float ang = (float)positions[t] * inv_freq[i];
    float s, c;
    sincosf(ang, &s, &c);
    cos_sin[idx] = make_float2(c, s);
}

// ---------------------------------------------------------------------------------------------
// For token t of request row_req[t] at position positions[t], with the row [q | k | v] =
// sum_p src[p][t]:  rotate every q head into q_out, and (when kv_pool is given) rotate every k head
// and store it together with v into the page block_table[req][pos / page_size] at slot
// pos % page_size.  Pairs are (i, i + half) for split-half and (2i, 2i + 1) for interleaved pairing
// (qwen_infer.c:782-790); features from rot on are copied.  src may be the partial sums of a
// split-K product.  The pool of one layer is [num_pages][2][nkv][page_size][hd].
// One rotated feature: me*cos - other*sin for the first of a pair, me*cos + other*sin for the second,
// with the rounding steps spelled out so that every kernel below gives the same bits.
__device__ __forceinline__ float rope_rotate(float me, float other, float2 f, bool first) {
    const float cross = __fmul_rn(other, f.y);
    return __fmaf_rn(me, f.x, first ? -cross : cross);
}

template <typename TS, typename TQ, typename TC>
__global__ void rope_kv_append_kernel(const TS* __restrict__ src, int src_stride, int parts, size_t part_stride,
                                      TQ* __restrict__ q_out, int q_stride, const float2* __restrict__ cos_sin,
                                      const int* __restrict__ positions, const int* __restrict__ row_req,
                                      const int* __restrict__ block_table, int max_pages,
                                      TC* __restrict__ kv_pool, int num_pages, int page_size,
                                      int nh, int nkv, int hd, int rot, int interleaved, unsigned* status) {
    extern __shared__ float row_s[];                 // the token's summed row [q | k | v]
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    const int half = rot >> 1;
    const int width = (nh + (kv_pool ? 2 * nkv : 0)) * hd;
    const TS* row = src + (size_t)t * src_stride;
    // the page of this token (independent of the row's values: in flight together with them)
    int page = 0, slot = 0;
    if (kv_pool) {
        const int pos = positions[t];
        page = block_table[(size_t)row_req[t] * max_pages + pos / page_size];
        slot = pos % page_size;
    }
    if (std::is_same<TS, float>::value && (width % 4 == 0) && (src_stride % 4 == 0) && (part_stride % 4 == 0) &&
        ((uintptr_t)src % 16 == 0)) {
        const float4* r4 = reinterpret_cast<const float4*>(row);
        for (int i = threadIdx.x; i < width / 4; i += blockDim.x)
            reinterpret_cast<float4*>(row_s)[i] = sum_parts4(r4 + i, parts, part_stride >> 2);
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) row_s[i] = sum_parts(row + i, parts, part_stride);
    }
    __syncthreads();
    const float2* cs = cos_sin ? cos_sin + (size_t)t * half : nullptr;
    auto rotated = [&](const float* head, int i) -> float {
        float me = head[i];
        if (i >= rot) return me;
        int pi, partner;
        bool first;
        if (interleaved) { pi = i >> 1; first = (i & 1) == 0; partner = first ? i + 1 : i - 1; }
        else { first = i < half; pi = first ? i : i - half; partner = first ? i + half : i - half; }
        float other = head[partner];
        return rope_rotate(me, other, cs[pi], first);
    };
    TQ* qo = q_out + (size_t)t * q_stride;
    for (int idx = threadIdx.x; idx < nh * hd; idx += blockDim.x) {
        int h = idx / hd, i = idx - h * hd;
        qo[idx] = from_float<TQ>(rotated(row_s + h * hd, i));
    }
    if (!kv_pool) return;
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0 && status) atomicOr(status, BG_STATUS_BAD_PAGE);
        return;
    }
    const float* k = row_s + nh * hd;
    const float* vv = k + nkv * hd;
    TC* kdst = kv_pool + ((size_t)page * 2 + 0) * nkv * page_size * hd;
    TC* vdst = kv_pool + ((size_t)page * 2 + 1) * nkv * page_size * hd;
    for (int idx = threadIdx.x; idx < nkv * hd; idx += blockDim.x) {
        int h = idx / hd, i = idx - h * hd;
        size_t dst = ((size_t)h * page_size + slot) * hd + i;
        vdst[dst] = from_float<TC>(vv[idx]);
        kdst[dst] = from_float<TC>(rotated(k + h * hd, i));
    }
}

// The common bfloat16 case (one tensor, split-half pairs over the whole head, head_dim a multiple of
// 16, bfloat16 cache): every thread rotates eight features of the first half of a head together with
// their eight partners, with 16-byte loads and stores and no staging in shared memory.
__global__ void __launch_bounds__(128)
rope_kv_append_bf16_kernel(const __nv_bfloat16* __restrict__ src, int src_stride, __nv_bfloat16* __restrict__ q_out,
                           int q_stride, const float2* __restrict__ cos_sin, const int* __restrict__ positions,
                           const int* __restrict__ row_req, const int* __restrict__ block_table, int max_pages,
                           __nv_bfloat16* __restrict__ kv_pool, int num_pages, int page_size, int nh, int nkv, int hd,
                           unsigned* status) {
    pdl_launch();
    const int t = blockIdx.x;
    const int half = hd >> 1, chunks = half >> 3;              // 8-feature chunks per half head
    const __nv_bfloat16* row = src + (size_t)t * src_stride;
    const float2* cs = cos_sin + (size_t)t * half;
    // where this token's key and value go: position and request are asked for before the wait for the kernel
    // ahead, the block-table entry once the first features are on their way, so that the chain of dependent
    // loads runs beside them instead of before them
    int pos = 0, rq = 0;
    if (kv_pool) { pos = positions[t]; rq = row_req[t]; }
    pdl_wait();
    int page = -2, slot = 0;                                   // -2: not looked up yet
    auto look_up = [&] {
        if (page != -2) return;
        page = -1;
        if (kv_pool) {
            page = block_table[(size_t)rq * max_pages + pos / page_size];
            slot = pos % page_size;
            if (page < 0 || page >= num_pages) {
                if (threadIdx.x == 0 && status) atomicOr(status, BG_STATUS_BAD_PAGE);
                page = -1;
            }
        }
    };
    const int n_heads = nh + (kv_pool ? nkv : 0);
    for (int item = threadIdx.x; item < n_heads * chunks; item += blockDim.x) {
        const int h = item / chunks, c = item - h * chunks;
        float a[8], b[8];
        load8(row + (size_t)h * hd + 8 * c, a);
        load8(row + (size_t)h * hd + half + 8 * c, b);
        float4 f4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) f4[i] = reinterpret_cast<const float4*>(cs + 8 * c)[i];
        look_up();
        float ra[8], rb[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float2 f = (i & 1) ? make_float2(f4[i >> 1].z, f4[i >> 1].w) : make_float2(f4[i >> 1].x, f4[i >> 1].y);
            ra[i] = rope_rotate(a[i], b[i], f, true);
            rb[i] = rope_rotate(b[i], a[i], f, false);
        }
        __nv_bfloat16* dst;
        if (h < nh) {
            dst = q_out + (size_t)t * q_stride + (size_t)h * hd;
        } else {
            if (page < 0) continue;
            dst = kv_pool + ((size_t)page * 2 + 0) * nkv * page_size * hd + ((size_t)(h - nh) * page_size + slot) * hd;
        }
        store8(dst + 8 * c, ra);
        store8(dst + half + 8 * c, rb);
    }
    look_up();
    if (kv_pool && page >= 0) {                                  // v: a plain copy
        const __nv_bfloat16* v = row + (size_t)(nh + nkv) * hd;
        __nv_bfloat16* vdst = kv_pool + ((size_t)page * 2 + 1) * nkv * page_size * hd;
        const int vc = hd >> 3;
        for (int item = threadIdx.x; item < nkv * vc; item += blockDim.x) {
            const int h = item / vc, c = item - h * vc;
            *reinterpret_cast<uint4*>(vdst + ((size_t)h * page_size + slot) * hd + 8 * c) =
                *reinterpret_cast<const uint4*>(v + (size_t)h * hd + 8 * c);
        }
    }
}

// For steps of few tokens: one block per (token, head) and one thread per feature, which sums its own
// value and its partner's from the partial sums directly.  Nothing is staged and nothing is waited for
// but the loads themselves, which are all in flight together.
template <typename TS, typename TQ, typename TC>
__global__ void rope_kv_append_heads_kernel(const TS* __restrict__ src, int src_stride, int parts, size_t part_stride,
                                            TQ* __restrict__ q_out, int q_stride, const float2* __restrict__ cos_sin,
                                            const int* __restrict__ positions, const int* __restrict__ row_req,
                                            const int* __restrict__ block_table, int max_pages,
                                            TC* __restrict__ kv_pool, int num_pages, int page_size,
                                            int nh, int nkv, int hd, int rot, int interleaved, unsigned* status) {
    pdl_launch();
    const int t = blockIdx.x, h = blockIdx.y, i = threadIdx.x;
    const int half = rot >> 1;
    const bool is_v = h >= nh + nkv;
    const TS* head = src + (size_t)t * src_stride + (size_t)h * hd;
    // where the key or value goes is known before the step began (positions and block tables are not written
    // by the kernels of a step): this chain of two loads runs while the kernel ahead finishes
    int page = 0, slot = 0;
    if (h >= nh) {
        const int pos = positions[t];
        page = block_table[(size_t)row_req[t] * max_pages + pos / page_size];
        slot = pos % page_size;
    }
    pdl_wait();
    if (i >= hd) return;               // (threads leave after the wait, not before it)
    float val = sum_parts(head + i, parts, part_stride);
    if (!is_v && i < rot) {
        int pi, partner;
        bool first;
        if (interleaved) { pi = i >> 1; first = (i & 1) == 0; partner = first ? i + 1 : i - 1; }
        else { first = i < half; pi = first ? i : i - half; partner = first ? i + half : i - half; }
        const float other = sum_parts(head + partner, parts, part_stride);
        val = rope_rotate(val, other, cos_sin[(size_t)t * half + pi], first);
    }
    if (h < nh) {
        q_out[(size_t)t * q_stride + (size_t)h * hd + i] = from_float<TQ>(val);
        return;
    }
    if (page < 0 || page >= num_pages) {
        if (i == 0 && status) atomicOr(status, BG_STATUS_BAD_PAGE);
        return;
    }
    const int kvh = is_v ? h - nh - nkv : h - nh;
    TC* dst = kv_pool + ((size_t)page * 2 + (is_v ? 1 : 0)) * nkv * page_size * hd + ((size_t)kvh * page_size + slot) * hd;
    dst[i] = from_float<TC>(val);
}

}  // namespace bg

using namespace bg;

extern "C" int bg_embed_gather(const void* table, int table_dtype, const int* ids, float* out, int T,
                               int d, int vocab, float scale, unsigned* status, cudaStream_t stream) {
    if (T <= 0) return BG_OK;
    BG_DISPATCH_DTYPE(table_dtype, TT, launch(embed_gather_kernel<TT>, dim3(T), dim3(256), 0, stream,
        (const TT*)table, ids, out, d, vocab, scale, status));
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_fill_normal(void* out, int out_dtype, long long n, unsigned long long key, long long first, float mean,
                              float std, cudaStream_t stream) {
    if (n <= 0) return BG_OK;
    const unsigned long long blocks = (unsigned long long)(n + 255) / 256;
    if (blocks > 0x7fffffffull) return BG_ERR_SHAPE;
    BG_DISPATCH_DTYPE(out_dtype, TO, launch(fill_normal_kernel<TO>, dim3((unsigned)blocks), dim3(256), 0, stream,
        (TO*)out, n, key, first, mean, std));
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_softcap(float* x, long long n, float cap, cudaStream_t stream) {
    if (n <= 0) return BG_OK;
    if (!(cap > 0.0f)) return BG_ERR_SHAPE;
    launch(softcap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, n, cap);
    BG_LAUNCH_CHECK();
    return BG_OK;
}

template <typename TD, typename TW, typename TO>
static int add_rmsnorm_launch(float* x, const void* delta, int parts, size_t part_stride, const void* w, float eps,
                              void* out, const int* rows, int n_rows, int d, int update, cudaStream_t stream) {
    size_t smem = (size_t)d * sizeof(float);
    if (smem > 200 * 1024) return BG_ERR_SHAPE;
    const bool vec = (d % 8 == 0) && (part_stride % 8 == 0) && ((uintptr_t)x % 16 == 0) && ((uintptr_t)delta % 16 == 0) &&
                     ((uintptr_t)w % 16 == 0) && ((uintptr_t)out % 16 == 0);
    if (vec && std::is_same<TD, float>::value && parts > 1 && !std::is_same<TO, float>::value && n_rows <= 64 && d <= 8192) {
        // few rows: clusters of 2, 4 or 8 CTAs per row, enough for about a wave of CTAs and for one chunk per thread
        int c = 2;
        while (c < 8 && (n_rows * c < 96 || (d / 4 + c - 1) / c > 256)) c *= 2;
        const int per = (d / 4 + c - 1) / c;
        if (per <= 256) {
            const dim3 grid(n_rows, 1, c), block((per + 31) / 32 * 32);
            cudaError_t e;
            if (c == 2) e = launch_cluster(add_rmsnorm_parts_cluster_kernel<TW, TO, 2>, grid, block, 0, stream, c, x, (const float*)delta, parts, part_stride, (const TW*)w, eps, (TO*)out, rows, d, update);
            else if (c == 4) e = launch_cluster(add_rmsnorm_parts_cluster_kernel<TW, TO, 4>, grid, block, 0, stream, c, x, (const float*)delta, parts, part_stride, (const TW*)w, eps, (TO*)out, rows, d, update);
            else e = launch_cluster(add_rmsnorm_parts_cluster_kernel<TW, TO, 8>, grid, block, 0, stream, c, x, (const float*)delta, parts, part_stride, (const TW*)w, eps, (TO*)out, rows, d, update);
            if (e != cudaSuccess) return (int)e;
            BG_LAUNCH_CHECK();
            return BG_OK;
        }
    }
    if (vec && std::is_same<TD, float>::value && parts > 1) {
        auto kern = add_rmsnorm_parts_kernel<TW, TO>;
        if (smem > BG_SMEM_OPT_IN) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        int threads = d / 4 >= 512 ? 512 : (d / 4 >= 256 ? 384 : 128);
        launch(kern, dim3(n_rows), dim3(threads), smem, stream, x, (const float*)delta, parts, part_stride, (const TW*)w, eps,
               (TO*)out, rows, d, update);
    } else if (vec && parts <= 1 && d <= 8 * 32 * 16 && n_rows >= 64 && !std::is_same<TO, float>::value) {
        // many rows of a bfloat16 step: a warp per row (2,048 rows of 1,536: 9.7 us against 11.0; for a handful of
        // rows the block per row below is the faster one: 2.9 against 6.8 us in a decoding step).  The float path
        // keeps ONE kernel for every number of rows, so that a row's statistics are summed in the same order
        // whatever else the step holds.
        const int iter = (d / 8 + 31) / 32;
        const unsigned blocks = (unsigned)((n_rows + 7) / 8);
#define BG_NORM_WARP(IT)                                                                                            \
        launch(add_rmsnorm_warp_kernel<TD, TW, TO, IT>, dim3(blocks), dim3(256), 0, stream, x, (const TD*)delta, (const TW*)w, \
               eps, (TO*)out, rows, n_rows, d, update)
        if (iter <= 2) BG_NORM_WARP(2);
        else if (iter <= 4) BG_NORM_WARP(4);
        else if (iter <= 8) BG_NORM_WARP(8);
        else BG_NORM_WARP(16);
#undef BG_NORM_WARP
    } else if (vec) {
        auto kern = add_rmsnorm_vec8_kernel<TD, TW, TO>;
        if (smem > BG_SMEM_OPT_IN) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        // as few trips through a row as 512 threads allow, and no thread without a chunk in the last trip
        const int d8 = d / 8, trips = (d8 + 511) / 512;
        int threads = (((d8 + trips - 1) / trips) + 31) / 32 * 32;
        if (threads < 64) threads = 64;
        launch(kern, dim3(n_rows), dim3(threads), smem, stream, x, (const TD*)delta, parts, part_stride, (const TW*)w, eps, (TO*)out,
                                                rows, d, update);
    } else {
        auto kern = add_rmsnorm_kernel<TD, TW, TO>;
        if (smem > BG_SMEM_OPT_IN) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch(kern, dim3(n_rows), dim3(256), smem, stream, x, (const TD*)delta, parts, part_stride, (const TW*)w, eps, (TO*)out, rows,
                                            d, update);
    }
    BG_LAUNCH_CHECK();
    return BG_OK;
}

template <typename TD, typename TW>
static int add_rmsnorm_out(float* x, const void* delta, int parts, size_t part_stride, const void* w, float eps, void* out,
                           int out_dtype, const int* rows, int n_rows, int d, int update, cudaStream_t stream) {
    if (out_dtype == BG_DTYPE_F32)
        return add_rmsnorm_launch<TD, TW, float>(x, delta, parts, part_stride, w, eps, out, rows, n_rows, d, update, stream);
    if (out_dtype == BG_DTYPE_BF16)
        return add_rmsnorm_launch<TD, TW, __nv_bfloat16>(x, delta, parts, part_stride, w, eps, out, rows, n_rows, d, update, stream);
    return BG_ERR_DTYPE;
}

// delta may be null (then delta_dtype is ignored) or [parts][T][d] with part_stride elements between
// parts; rows may be null (then row r reads source row r).
extern "C" int bg_add_rmsnorm(float* x, const void* delta, int delta_dtype, int parts, long long part_stride,
                              const void* w, int w_dtype, float eps, void* out, int out_dtype, const int* rows,
                              int n_rows, int d, int update, cudaStream_t stream) {
    if (n_rows <= 0) return BG_OK;
    if (!delta) { delta_dtype = BG_DTYPE_F32; parts = 0; }
    BG_DISPATCH_DTYPE(delta_dtype, TD, BG_DISPATCH_DTYPE(w_dtype, TW,
        return (add_rmsnorm_out<TD, TW>(x, delta, parts, (size_t)part_stride, w, eps, out, out_dtype, rows, n_rows, d,
                                        update, stream))));
    return BG_OK;
}

extern "C" int bg_add_residual(float* x, const void* delta, int delta_dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return BG_OK;
    unsigned blocks = (unsigned)((n + 255) / 256);
    BG_DISPATCH_DTYPE(delta_dtype, TD, launch(add_residual_kernel<TD>, dim3(blocks), dim3(256), 0, stream, x, (const TD*)delta, (size_t)n));
    BG_LAUNCH_CHECK();
    return BG_OK;
}

template <typename TI>
static int swiglu_in(const void* gu, int parts, size_t part_stride, void* out, int out_dtype, int rows, int im, int block,
                     cudaStream_t stream) {
    const bool small = (size_t)rows * (size_t)im < (1ull << 32);          // the vector kernels count their pieces in 32 bits
    const bool vec = small && parts == 1 && (im % 8 == 0) && (block % 8 == 0) && ((uintptr_t)gu % 16 == 0) && ((uintptr_t)out % 16 == 0);
    if (vec) {
        size_t total = (size_t)rows * (im / 8);
        unsigned blocks = (unsigned)((total + 255) / 256);
        BG_DISPATCH_DTYPE(out_dtype, TO, launch(swiglu_vec8_kernel<TI, TO>, dim3(blocks), dim3(256), 0, stream,
            (const TI*)gu, (TO*)out, rows, im, block));
    } else if (small && std::is_same<TI, float>::value && (im % 4 == 0) && (block % 4 == 0) && (part_stride % 4 == 0) &&
               ((uintptr_t)gu % 16 == 0) && ((uintptr_t)out % 16 == 0)) {
        size_t total = (size_t)rows * (im / 4);
        unsigned blocks = (unsigned)((total + 255) / 256);
        BG_DISPATCH_DTYPE(out_dtype, TO, launch(swiglu_parts_vec4_kernel<TO>, dim3(blocks), dim3(256), 0, stream,
            (const float*)gu, parts, part_stride, (TO*)out, rows, im, block));
    } else {
        size_t total = (size_t)rows * im;
        unsigned blocks = (unsigned)((total + 255) / 256);
        BG_DISPATCH_DTYPE(out_dtype, TO, launch(swiglu_kernel<TI, TO>, dim3(blocks), dim3(256), 0, stream,
            (const TI*)gu, parts, part_stride, (TO*)out, rows, im, block));
    }
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_swiglu(const void* gu, int in_dtype, int parts, long long part_stride, void* out, int out_dtype,
                         int rows, int im, int block, cudaStream_t stream) {
    if (rows <= 0) return BG_OK;
    if (parts < 1 || block < 0 || (block > 0 && im % block != 0)) return BG_ERR_SHAPE;
    BG_DISPATCH_DTYPE(in_dtype, TI, return (swiglu_in<TI>(gu, parts, (size_t)part_stride, out, out_dtype, rows, im, block, stream)));
    return BG_OK;
}

extern "C" int bg_rope_table(const int* positions, const float* inv_freq, float* cos_sin, int T, int half,
                             cudaStream_t stream) {
    if (T <= 0 || half <= 0) return BG_OK;
    int total = T * half;
    launch(rope_table_kernel, dim3((total + 255) / 256), dim3(256), 0, stream, positions, inv_freq, (float2*)cos_sin, T, half);
    BG_LAUNCH_CHECK();
    return BG_OK;
}

template <typename TS, typename TQ>
static int rope_kv_cache(const void* src, int src_stride, int parts, size_t part_stride, void* q_out, int q_stride,
                         const float* cos_sin, const int* positions, const int* row_req, const int* block_table,
                         int max_pages, void* kv_pool, int cache_dtype, int num_pages, int page_size, int T, int nh,
                         int nkv, int hd, int rot, int interleaved, unsigned* status, cudaStream_t stream) {
    // one block per token stages the token's whole q/k/v row in shared memory; a row that does not fit there
    // (many wide heads in float) goes head by head, like the steps of few tokens
    const size_t smem = (size_t)(nh + 2 * nkv) * hd * sizeof(float);
    const bool row_fits = smem <= 200 * 1024;
    if (!row_fits && hd > 1024) return BG_ERR_SHAPE;
    if ((T <= 64 || !row_fits) && hd <= 1024) {
        dim3 grid(T, nh + (kv_pool ? 2 * nkv : 0));
        BG_DISPATCH_DTYPE(cache_dtype, TC, launch(rope_kv_append_heads_kernel<TS, TQ, TC>, grid, dim3((hd + 31) / 32 * 32), 0,
            stream, (const TS*)src, src_stride, parts, part_stride, (TQ*)q_out, q_stride, (const float2*)cos_sin, positions,
            row_req, block_table, max_pages, (TC*)kv_pool, num_pages, page_size, nh, nkv, hd, rot, interleaved, status));
        BG_LAUNCH_CHECK();
        return BG_OK;
    }
    if (smem > BG_SMEM_OPT_IN) {
        BG_DISPATCH_DTYPE(cache_dtype, TC, cudaFuncSetAttribute(rope_kv_append_kernel<TS, TQ, TC>,
            cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    }
    BG_DISPATCH_DTYPE(cache_dtype, TC, launch(rope_kv_append_kernel<TS, TQ, TC>, dim3(T), dim3(256), smem, stream,
        (const TS*)src, src_stride, parts, part_stride, (TQ*)q_out, q_stride, (const float2*)cos_sin, positions, row_req,
        block_table, max_pages, (TC*)kv_pool, num_pages, page_size, nh, nkv, hd, rot, interleaved, status));
    BG_LAUNCH_CHECK();
    return BG_OK;
}

template <typename TS>
static int rope_kv_q(const void* src, int src_stride, int parts, size_t part_stride, void* q_out, int q_dtype, int q_stride,
                     const float* cos_sin, const int* positions, const int* row_req, const int* block_table,
                     int max_pages, void* kv_pool, int cache_dtype, int num_pages, int page_size, int T, int nh, int nkv,
                     int hd, int rot, int interleaved, unsigned* status, cudaStream_t stream) {
    BG_DISPATCH_DTYPE(q_dtype, TQ, return (rope_kv_cache<TS, TQ>(src, src_stride, parts, part_stride, q_out, q_stride,
        cos_sin, positions, row_req, block_table, max_pages, kv_pool, cache_dtype, num_pages, page_size, T, nh, nkv, hd,
        rot, interleaved, status, stream)));
    return BG_OK;
}

// src rows are [q | k | v] (or only q when kv_pool is null: a mixer that reads another stage's
// cache).  q_out must not alias src.
extern "C" int bg_rope_kv_append(const void* src, int src_dtype, int src_stride, int parts, long long part_stride,
                                 void* q_out, int q_dtype, int q_stride, const float* cos_sin, const int* positions,
                                 const int* row_req, const int* block_table, int max_pages, void* kv_pool,
                                 int cache_dtype, int num_pages, int page_size, int T, int nh, int nkv, int hd,
                                 int rot, int interleaved, unsigned* status, cudaStream_t stream) {
    if (T <= 0) return BG_OK;
    if (rot < 0 || rot > hd || (rot & 1) || parts < 1) return BG_ERR_SHAPE;
    if (rot > 0 && !cos_sin) return BG_ERR_SHAPE;
    if (src_dtype == BG_DTYPE_BF16 && q_dtype == BG_DTYPE_BF16 && (!kv_pool || cache_dtype == BG_DTYPE_BF16) && parts == 1 &&
        !interleaved && rot == hd && hd % 16 == 0 && src_stride % 8 == 0 && q_stride % 8 == 0 &&
        (uintptr_t)src % 16 == 0 && (uintptr_t)q_out % 16 == 0 && (uintptr_t)kv_pool % 16 == 0) {
        launch(rope_kv_append_bf16_kernel, dim3(T), dim3(128), 0, stream, (const __nv_bfloat16*)src, src_stride,
               (__nv_bfloat16*)q_out, q_stride, (const float2*)cos_sin, positions, row_req, block_table, max_pages,
               (__nv_bfloat16*)kv_pool, num_pages, page_size, nh, nkv, hd, status);
        BG_LAUNCH_CHECK();
        return BG_OK;
    }
    if (!kv_pool) cache_dtype = BG_DTYPE_F32;
    BG_DISPATCH_DTYPE(src_dtype, TS, return (rope_kv_q<TS>(src, src_stride, parts, (size_t)part_stride, q_out, q_dtype,
        q_stride, cos_sin, positions, row_req, block_table, max_pages, kv_pool, cache_dtype, num_pages, page_size, T, nh,
        nkv, hd, rot, interleaved, status, stream)));
    return BG_OK;
}
