// Sampling from float logits [n, V]: the index of the first maximum (qwen_infer.c:2152-2155), or a
// draw from softmax(logits / T) by inverting the cumulative distribution in index order with a
// uniform number that the host supplies per row.  One block per row; the order of every sum is
// fixed by V and the block size alone.
#include "common.cuh"

namespace bg {

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ void argmax_combine(float& v, int& i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

// first index of the maximum of row[0..V); NaN never wins
__device__ int block_argmax(const float* row, int V, float* s_val, int* s_idx, float* max_out) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        float v = row[i];
        if (v > best || (bi == 0x7fffffff && v == best)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        argmax_combine(best, bi, ov, oi);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        int nw = (blockDim.x + 31) >> 5;
        best = lane < nw ? s_val[lane] : -INFINITY;
        bi = lane < nw ? s_idx[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, best, o);
            int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            argmax_combine(best, bi, ov, oi);
        }
        if (lane == 0) { s_val[0] = best; s_idx[0] = bi; }
    }
    __syncthreads();
    *max_out = s_val[0];
    int r = s_idx[0];
    __syncthreads();
    return r == 0x7fffffff ? 0 : r;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
              const float* __restrict__ uniform, int* __restrict__ out) {
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    __shared__ float s_chunk[SAMPLE_THREADS];
    __shared__ int s_pick;
    __shared__ float s_before;
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * V;
    float mx;
    const int am = block_argmax(row, V, s_val, s_idx, &mx);
    const float T = temperature ? temperature[r] : 0.0f;
    if (!(T > 0.0f)) {
        if (threadIdx.x == 0) out[r] = am;
        return;
    }
    // contiguous chunk of each thread, so that the cumulative sum runs in index order
    const int per = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int b = threadIdx.x * per, e = min(V, b + per);
    const float invT = 1.0f / T;
    float cs = 0.0f;
    for (int i = b; i < e; ++i) cs += expf((row[i] - mx) * invT);
    s_chunk[threadIdx.x] = cs;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.0f;
        for (int i = 0; i < SAMPLE_THREADS; ++i) total += s_chunk[i];
        const float target = uniform[r] * total;
        float run = 0.0f;
        int pick = -1;
        for (int i = 0; i < SAMPLE_THREADS; ++i) {
            if (s_chunk[i] > 0.0f && run + s_chunk[i] > target) { pick = i; break; }
            run += s_chunk[i];
        }
        s_pick = pick;
        s_before = run;
        if (pick < 0) out[r] = am;          // rounding pushed the target past the total: take the mode
        else s_before = run;
    }
    __syncthreads();
    if (s_pick == (int)threadIdx.x) {
        float total = 0.0f;
        for (int i = 0; i < SAMPLE_THREADS; ++i) total += s_chunk[i];
        const float target = uniform[r] * total;
        float run = s_before;
        int pick = -1, last = b;
        for (int i = b; i < e; ++i) {
            float pe = expf((row[i] - mx) * invT);
            if (pe > 0.0f) last = i;
            run += pe;
            if (run > target) { pick = i; break; }
        }
        out[r] = pick >= 0 ? pick : last;
    }
}

}  // namespace bg

// temperature may be null (all rows greedy); uniform may be null only then.
extern "C" int bg_sample(const float* logits, int n, int V, const float* temperature, const float* uniform, int* out,
                         cudaStream_t stream) {
    if (n <= 0) return BG_OK;
    if (V <= 0) return BG_ERR_SHAPE;
    if (temperature && !uniform) return BG_ERR_SHAPE;
    bg::sample_kernel<<<n, bg::SAMPLE_THREADS, 0, stream>>>(logits, V, temperature, uniform, out);
    BG_LAUNCH_CHECK();
    return BG_OK;
}
