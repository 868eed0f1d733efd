// Sampling from float logits [n, V]: the index of the first maximum (qwen_infer.c:2152-2155), or a
// draw from softmax(logits / T) by inverting the cumulative distribution in index order with a
// uniform number that the host supplies per row.  One block per row; the order of every sum is
// fixed by V and the block size alone.
#include "common.cuh"

namespace bg {


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

// ---- two stages, so that a row of a large vocabulary is spread over many blocks
constexpr int SAMPLE_CHUNKS = 64;        // blocks per row in stage 1
constexpr int STAGE_THREADS = 256;

// Stage 1: block (row, chunk) finds the first maximum of its chunk and, for a row with a positive
// temperature, the sum of exp((x - chunk max) / T) over the chunk.
__global__ void __launch_bounds__(STAGE_THREADS)
sample_stage1_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
                     float* __restrict__ c_max, int* __restrict__ c_arg, float* __restrict__ c_sum) {
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    __shared__ float red[32];
    pdl_launch();
    pdl_wait();
    const int r = blockIdx.x, c = blockIdx.y;
    const int per = (V + SAMPLE_CHUNKS - 1) / SAMPLE_CHUNKS;
    const int b = c * per, e = min(V, b + per);
    const float* row = logits + (size_t)r * V;
    float mx = -INFINITY;
    int am = 0x7fffffff;
    if (b < e) {
        am = b + block_argmax(row + b, e - b, s_val, s_idx, &mx);
    }
    const float T = temperature ? temperature[r] : 0.0f;
    float sum = 0.0f;
    if (T > 0.0f && b < e) {
        const float invT = 1.0f / T;
        // contiguous sub-chunks per thread keep the order of the sum fixed
        const int sub = (e - b + STAGE_THREADS - 1) / STAGE_THREADS;
        const int sb = b + threadIdx.x * sub, se = min(e, sb + sub);
        float part = 0.0f;
        for (int i = sb; i < se; ++i) part += expf((row[i] - mx) * invT);
        sum = block_sum(part, red);
    }
    if (threadIdx.x == 0) {
        c_max[r * SAMPLE_CHUNKS + c] = mx;
        c_arg[r * SAMPLE_CHUNKS + c] = am;
        c_sum[r * SAMPLE_CHUNKS + c] = sum;
    }
}

// Stage 2: one block per row joins the chunks.  Greedy: the first maximum.  Otherwise the chunk in
// which the cumulative sum passes u * total, then the index inside it.
__global__ void __launch_bounds__(STAGE_THREADS)
sample_stage2_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
                     const float* __restrict__ uniform, const float* __restrict__ c_max, const int* __restrict__ c_arg,
                     const float* __restrict__ c_sum, int* __restrict__ out, int* __restrict__ feed_tokens,
                     int* __restrict__ feed_positions, const int* __restrict__ advance) {
    __shared__ float s_part[STAGE_THREADS];
    __shared__ float s_gmax, s_target, s_before;
    __shared__ int s_chunk, s_pick;
    pdl_launch();
    pdl_wait();
    const int r = blockIdx.x;
    const float T = temperature ? temperature[r] : 0.0f;
    // The chosen token; for a decoding loop that runs on the device it also becomes the row's next input token, and
    // the row's position moves on by advance[r] (0 for a row that pads the batch).
    auto emit = [&](int token) {
        out[r] = token;
        if (feed_tokens) feed_tokens[r] = token;
        if (feed_positions) feed_positions[r] += advance ? advance[r] : 1;
    };
    if (threadIdx.x == 0) {
        float g = -INFINITY;
        int arg = 0;
        for (int c = 0; c < SAMPLE_CHUNKS; ++c) {
            float v = c_max[r * SAMPLE_CHUNKS + c];
            if (v > g) { g = v; arg = c_arg[r * SAMPLE_CHUNKS + c]; }       // strict: the first maximum wins
        }
        s_gmax = g;
        s_pick = (arg == 0x7fffffff) ? 0 : arg;
        s_chunk = -1;
        if (T > 0.0f) {
            const float invT = 1.0f / T;
            float total = 0.0f;
            for (int c = 0; c < SAMPLE_CHUNKS; ++c) {
                float cm = c_max[r * SAMPLE_CHUNKS + c];
                if (cm > -INFINITY) total += c_sum[r * SAMPLE_CHUNKS + c] * expf((cm - g) * invT);
            }
            const float target = uniform[r] * total;
            float run = 0.0f;
            int last = -1;
            for (int c = 0; c < SAMPLE_CHUNKS; ++c) {
                float cm = c_max[r * SAMPLE_CHUNKS + c];
                float cs = (cm > -INFINITY) ? c_sum[r * SAMPLE_CHUNKS + c] * expf((cm - g) * invT) : 0.0f;
                if (cs > 0.0f) last = c;
                if (cs > 0.0f && run + cs > target) { s_chunk = c; break; }
                run += cs;
            }
            if (s_chunk < 0) { s_chunk = last; run = INFINITY; }      // rounding pushed the target past the total
            s_target = target;
            s_before = run;
        }
    }
    __syncthreads();
    if (!(T > 0.0f) || s_chunk < 0) {
        if (threadIdx.x == 0) emit(s_pick);
        return;
    }
    const float* row = logits + (size_t)r * V;
    const int per = (V + SAMPLE_CHUNKS - 1) / SAMPLE_CHUNKS;
    const int b = s_chunk * per, e = min(V, b + per);
    const float invT = 1.0f / T, g = s_gmax;
    const int sub = (e - b + STAGE_THREADS - 1) / STAGE_THREADS;
    const int sb = b + threadIdx.x * sub, se = min(e, sb + sub);
    float part = 0.0f;
    for (int i = sb; i < se; ++i) part += expf((row[i] - g) * invT);
    s_part[threadIdx.x] = part;
    __syncthreads();
    if (threadIdx.x == 0) {
        float run = s_before == INFINITY ? -INFINITY : s_before;
        int owner = -1, last = 0;
        for (int i = 0; i < STAGE_THREADS; ++i) {
            if (s_part[i] > 0.0f) last = i;
            if (s_part[i] > 0.0f && run + s_part[i] > s_target) { owner = i; break; }
            run += s_part[i];
        }
        if (owner < 0) { owner = last; run = -INFINITY; }
        // the index inside the owner's sub-chunk
        const int ob = b + owner * sub, oe = min(e, ob + sub);
        int pick = -1, lastnz = ob;
        for (int i = ob; i < oe; ++i) {
            float pe = expf((row[i] - g) * invT);
            if (pe > 0.0f) lastnz = i;
            run += pe;
            if (run > s_target) { pick = i; break; }
        }
        emit(pick >= 0 ? pick : lastnz);
    }
}

}  // namespace bg

// Bytes of scratch that bg_sample needs for n rows.
extern "C" long long bg_sample_scratch_bytes(int n) { return (long long)n * bg::SAMPLE_CHUNKS * 12; }

// temperature may be null (all rows greedy); uniform may be null only then.  scratch holds
// bg_sample_scratch_bytes(n) bytes.  feed_tokens [n] and feed_positions [n] (either may be null) are the input buffers
// of a decoding step that is replayed: the chosen token is also written to feed_tokens[r], and feed_positions[r]
// grows by advance[r] (by 1 where advance is null).
extern "C" int bg_sample_feed(const float* logits, int n, int V, const float* temperature, const float* uniform, int* out,
                              void* scratch, int* feed_tokens, int* feed_positions, const int* advance, cudaStream_t stream) {
    if (n <= 0) return BG_OK;
    if (V <= 0) return BG_ERR_SHAPE;
    if (temperature && !uniform) return BG_ERR_SHAPE;
    if (!scratch) return BG_ERR_SHAPE;
    float* c_max = (float*)scratch;
    int* c_arg = (int*)(c_max + (size_t)n * bg::SAMPLE_CHUNKS);
    float* c_sum = (float*)(c_arg + (size_t)n * bg::SAMPLE_CHUNKS);
    dim3 grid(n, bg::SAMPLE_CHUNKS);
    bg::launch(bg::sample_stage1_kernel, grid, dim3(bg::STAGE_THREADS), 0, stream, logits, V, temperature, c_max, c_arg, c_sum);
    BG_LAUNCH_CHECK();
    bg::launch(bg::sample_stage2_kernel, dim3(n), dim3(bg::STAGE_THREADS), 0, stream, logits, V, temperature, uniform, c_max, c_arg, c_sum, out,
               feed_tokens, feed_positions, advance);
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_sample(const float* logits, int n, int V, const float* temperature, const float* uniform, int* out,
                         void* scratch, cudaStream_t stream) {
    return bg_sample_feed(logits, n, V, temperature, uniform, out, scratch, nullptr, nullptr, nullptr, stream);
}
