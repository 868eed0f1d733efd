// The product of a step of few tokens (up to 64) with what stands before and behind it fused in, on
// the fifth-generation tensor cores:
//
//   acc[t, n] = sum_k X[t, k] * W[n, k]        W: [n_out, K] bfloat16 by TMA, 128 output features per CTA
//
//   X         either bfloat16 activations by TMA, or made here from the float residual stream:
//             X[t, k] = bf16(x[t, k] * rstd[t] * g[k]) with rstd[t] = 1 / sqrt(ssq[t] / K + eps), where
//             ssq[t] is the sum (in index order) of partial sums of squares that the kernel which wrote
//             x left behind.  That is RMSNorm (qwen_infer.c:689-704) without a kernel of its own: the
//             four warps that later run the epilogue make the operand tiles, stage by stage.
//   split-K   blockIdx.z takes a range of 64-wide k-blocks; the CTAs of one output tile form a thread
//             block cluster (1, 1, splits).  Rank r owns 128 / splits rows of the tile: every CTA stores
//             those rows of its accumulator into rank r's shared memory (distributed shared memory), the
//             cluster meets at ONE barrier, and rank r adds the parts up in rank order.  No partial sums
//             go to global memory, and the order of the sum is fixed by the shapes.
//   epilogue  plain:    out[t, n] = acc (+ bias[n]), float or bfloat16;
//             residual: x[t, n] += acc (+ bias[n]) in the float residual stream, and the sums of squares
//                       of the new x over the CTA's rows go to ssq_out[part][t] (for the next norm);
//             swiglu:   W's rows are interleaved, 64 of the gate then the 64 of up that belong to them:
//                       h[t, 64 * tile + i] = silu(acc[i]) * acc[64 + i] as bfloat16
//                       (qwen_infer.c:727-733), so gate_up never reaches global memory;
//             rope:     W's rows are [query heads | key heads | value heads] of hd features (hd 32, 64 or 128):
//                       queries and keys are rotated by their token's angles (feature d with d + hd / 2,
//                       qwen_infer.c:782-790), queries go to q[t, :] as bfloat16, keys and values into the
//                       cache page and slot of their token's position, so q/k/v never reach global memory
//                       as one row and the step has no kernel for rotation and append.
//
// Every wait on an mbarrier is bounded and records BG_STATUS_TIMEOUT; a CTA that gave up still goes
// through the cluster's barriers, so its peers do not wait for it.
#include <type_traits>

#include "tc_common.cuh"

namespace bg {

constexpr int GF_PLAIN = 0, GF_RESIDUAL = 1, GF_SWIGLU = 2, GF_ROPE = 3;
constexpr int SSQ_AHEAD = 24;        // partial sums of squares that a thread of the norm prologue asks for at a time

struct FusedParams {
    // the operand made from the residual stream (xf == null: X comes by TMA)
    const float* xf;
    int ldxf;
    const float* ssq_in;            // [n_ssq_in][ssq_in_stride]
    int n_ssq_in, ssq_in_stride;
    const __nv_bfloat16* norm_w;    // [K]
    float eps;
    // the epilogue
    const float* bias;              // [n_out] or null
    int mode;
    void* out;                      // plain: [T][ldo]; residual: the float stream [T][ldo]; swiglu: bfloat16 [T][ldo]
    int out_dtype, ldo;
    float* ssq_out;                 // residual: [tiles * splits][ssq_out_stride]
    int ssq_out_stride;
    int n_out, T, K, kb_per_split, splits;
    int log_splits;                 // splits is a power of two: divisions by it and by the rows of a rank are shifts
    // swiglu and rope work on pairs of rows of the tile, 1 << pair_log apart (gate i and up 64 + i; feature d of a
    // head and d + hd / 2): a rank owns both rows of its 64 / splits pairs
    int pair_log;
    unsigned* status;
};

// What the rope mode needs beside: out is q [T][ldo] bfloat16.  (A parameter of its own, which the kernels of the other
// modes do not carry.)
struct RopeParams {
    const float2* cos_sin;          // [T][hd / 2] (cos, sin) of each row's position
    const int* positions;           // [T]
    const int* row_req;             // [T] row of the block table
    const int* block_table;         // [requests][max_pages]
    __nv_bfloat16* kv_pool;         // [num_pages][2][nkv][page_size][hd]
    int max_pages, num_pages, page_size, nh, nkv;
};
struct NoRope {};

// Pair j of a tile is rows row_of_pair(j) and row_of_pair(j) + (1 << pair_log).
__device__ __forceinline__ int pair_of_row(int m, int pair_log) { return ((m >> (pair_log + 1)) << pair_log) | (m & ((1 << pair_log) - 1)); }
__device__ __forceinline__ int side_of_row(int m, int pair_log) { return (m >> pair_log) & 1; }
__device__ __forceinline__ int row_of_pair(int j, int pair_log) { return ((j >> pair_log) << (pair_log + 1)) | (j & ((1 << pair_log) - 1)); }

// The sum of the S ranks' parts of one value, in rank order (S is 1, 2, 4, 8 or 16; the loads of a sum go out together).
template <int S_>
__device__ __forceinline__ float ranks_sum_of(const float* rp, int part) {
    float a[S_];
#pragma unroll
    for (int s = 0; s < S_; ++s) a[s] = rp[s * part];
    float v = a[0];
#pragma unroll
    for (int s = 1; s < S_; ++s) v += a[s];
    return v;
}
__device__ __forceinline__ float ranks_sum(const float* rp, int part, int S) {
    switch (S) {
        case 1: return rp[0];
        case 2: return ranks_sum_of<2>(rp, part);
        case 4: return ranks_sum_of<4>(rp, part);
        case 8: return ranks_sum_of<8>(rp, part);
        default: return ranks_sum_of<16>(rp, part);
    }
}

__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;\n" ::: "memory"); }   // warps 2..5

// ROPE: the kernel of the rope mode is an instance of its own, so that the other modes' code (and what the compiler
// makes of it) does not change with it.
template <int BN, int STAGES, bool ROPE>
__global__ void __launch_bounds__(TC_THREADS)
gemm_fused_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, FusedParams p,
                  typename std::conditional<ROPE, RopeParams, NoRope>::type r) {
    constexpr unsigned A_BYTES = TC_BM * TC_BK * 2;
    constexpr unsigned B_BYTES = BN * TC_BK * 2;
    constexpr unsigned STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr unsigned TMEM_COLS = BN < 32 ? 32 : BN;
    constexpr int CHUNKS = BN * 8 / 128;                 // 16-byte pieces of an operand tile per epilogue thread
    extern __shared__ unsigned char gf_smem_raw[];
    unsigned char* tiles = (unsigned char*)(((uintptr_t)gf_smem_raw + 1023) & ~(uintptr_t)1023);
    // what the ranks of the cluster send to this one: [rank][token][row of this rank's share]; it is written by
    // peers while this CTA may still be in its main loop, so it has shared memory of its own
    float* recv = reinterpret_cast<float*>(tiles + (size_t)STAGES * STAGE_BYTES);
    float* sq = reinterpret_cast<float*>(tiles);                           // [BN][rows of this rank], over the stages once they are done
    __shared__ __align__(8) unsigned long long full_bar[STAGES];
    __shared__ __align__(8) unsigned long long empty_bar[STAGES];
    __shared__ __align__(8) unsigned long long acc_bar;
    __shared__ unsigned tmem_base_sh;
    __shared__ int failed;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_m = blockIdx.x, tile_n = blockIdx.y, split = blockIdx.z;    // split == rank in the cluster
    const int n_kb_total = (p.K + TC_BK - 1) / TC_BK;
    const int kb0 = split * p.kb_per_split;
    const int n_kb = min(p.kb_per_split, n_kb_total - kb0);
    const bool make_x = p.xf != nullptr;

    pdl_launch();
    // The cluster's barrier is used twice.  First: every thread arrives here and waits before anything is stored
    // into a peer's shared memory, so that every CTA of the cluster is known to be running by then.
    if (p.splits > 1) cluster_arrive_relaxed();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], make_x ? 5 : 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&acc_bar, 1);
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(&tmem_base_sh)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = tmem_base_sh;

    // What the reduction at the end adds to the product (the bias of this thread's row; in residual mode the
    // stream's values that it will update) is asked for while the main loop still runs: up to four values.
    // (rope: the two biases and the angle's cosine and sine for the thread's first token, and where that token's key
    // or value goes)
    float pre_bias = 0.0f, pre_x[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    int pre_page = 0, pre_slot = 0;

    if (warp == 0) {
        // ---------------- TMA producer: the weights (requested before the kernel ahead has finished) and,
        // when they come by TMA, the activations
        if (lane == 0 && n_kb > 0) {
            const unsigned stage_tx = make_x ? A_BYTES : STAGE_BYTES;
            const int ahead = n_kb < STAGES ? n_kb : STAGES;
            for (int i = 0; i < ahead; ++i) {
                mbar_expect_tx(&full_bar[i], stage_tx);
                tma_load_2d(tiles + (size_t)i * STAGE_BYTES, &map_w, (kb0 + i) * TC_BK, tile_m * TC_BM, &full_bar[i]);
            }
            pdl_wait();
            if (!make_x)
                for (int i = 0; i < ahead; ++i)
                    tma_load_2d(tiles + (size_t)i * STAGE_BYTES + A_BYTES, &map_x, (kb0 + i) * TC_BK, tile_n * BN, &full_bar[i]);
            for (int i = ahead; i < n_kb; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(&empty_bar[s], ((i / STAGES) - 1) & 1)) { atomicExch(&failed, 1); break; }
                unsigned char* a = tiles + (size_t)s * STAGE_BYTES;
                mbar_expect_tx(&full_bar[s], stage_tx);
                tma_load_2d(a, &map_w, (kb0 + i) * TC_BK, tile_m * TC_BM, &full_bar[s]);
                if (!make_x) tma_load_2d(a + A_BYTES, &map_x, (kb0 + i) * TC_BK, tile_n * BN, &full_bar[s]);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer
        if (lane == 0 && n_kb > 0) {
            constexpr unsigned idesc = instr_desc_bf16(TC_BM, BN < 16 ? 16 : BN);
            bool ok = true;
            for (int i = 0; i < n_kb && ok; ++i) {
                const int s = i % STAGES;
                ok = mbar_wait(&full_bar[s], (i / STAGES) & 1);
                if (!ok) { atomicExch(&failed, 1); break; }
                tc_fence_after();
                const unsigned a_addr = smem_u32(tiles + (size_t)s * STAGE_BYTES);
                const unsigned b_addr = a_addr + A_BYTES;
#pragma unroll
                for (int k = 0; k < TC_BK / 16; ++k)
                    tc_mma(tmem_base, smem_desc_sw128(a_addr + k * 32), smem_desc_sw128(b_addr + k * 32), idesc,
                           (i > 0 || k > 0) ? 1u : 0u);
                tc_commit(&empty_bar[s]);
            }
            tc_commit(&acc_bar);
        }
    } else {
        // ---------------- warps 2..5: first the operand tiles from the residual stream, then the epilogue
        const int te = threadIdx.x - 64;                                   // 0..127
        const int quarter = warp & 3;                                      // the tensor-memory lanes of this warp
        bool ok = true;
        pdl_wait();
        if (make_x && n_kb > 0) {
            // thread te makes pieces te, te + 128, ...: piece e is token e / 8 of the tile, features 8 (e % 8) ..+7
            float rstd[CHUNKS];
            const float* xrow[CHUNKS];
            const int c8 = te & 7;
#pragma unroll
            for (int j = 0; j < CHUNKS; ++j) {
                // the eight threads of a token share the parts of its sum of squares: thread c8 adds parts c8,
                // c8 + 8, ... (SSQ_AHEAD loads on their way at a time: the parts that a product over 16 ranges of K and
                // 12 tiles leaves come in one trip to L2), then the eight sums meet in a fixed order
                const int t = tile_n * BN + (te + j * 128) / 8;
                float ssq = 0.0f;
                if (t < p.T) {
                    for (int q = c8; q < p.n_ssq_in; q += 8 * SSQ_AHEAD) {
                        float a[SSQ_AHEAD];
#pragma unroll
                        for (int u = 0; u < SSQ_AHEAD; ++u)
                            a[u] = q + 8 * u < p.n_ssq_in ? p.ssq_in[(size_t)(q + 8 * u) * p.ssq_in_stride + t] : 0.0f;
#pragma unroll
                        for (int u = 0; u < SSQ_AHEAD; u += 4) ssq += (a[u] + a[u + 1]) + (a[u + 2] + a[u + 3]);
                    }
                }
                ssq += __shfl_xor_sync(0xffffffffu, ssq, 1);
                ssq += __shfl_xor_sync(0xffffffffu, ssq, 2);
                ssq += __shfl_xor_sync(0xffffffffu, ssq, 4);
                rstd[j] = t < p.T ? 1.0f / sqrtf(ssq / (float)p.K + p.eps) : 0.0f;
                xrow[j] = p.xf + (size_t)(t < p.T ? t : 0) * p.ldxf;
            }
            // the values of DEPTH k-blocks are on their way at any time: a k-block costs one trip to L2, and
            // one at a time would make the operand tiles slower than the weights arrive
            constexpr int DEPTH = CHUNKS == 1 ? 4 : (CHUNKS == 2 ? 2 : 1);
            float v[DEPTH][CHUNKS][8], g[DEPTH][8];
            auto fetch = [&](int i, int slot) {
                const int k = (kb0 + i) * TC_BK + c8 * 8;
#pragma unroll
                for (int q = 0; q < 8; ++q) g[slot][q] = 0.0f;
                if (i < n_kb && k < p.K) load8(p.norm_w + k, g[slot]);     // K is a multiple of 8
#pragma unroll
                for (int j = 0; j < CHUNKS; ++j) {
#pragma unroll
                    for (int q = 0; q < 8; ++q) v[slot][j][q] = 0.0f;
                    if (i < n_kb && k < p.K && rstd[j] != 0.0f) load8(xrow[j] + k, v[slot][j]);
                }
            };
#pragma unroll
            for (int d = 0; d < DEPTH; ++d) fetch(d, d);
            for (int i0 = 0; i0 < n_kb && ok; i0 += DEPTH) {
#pragma unroll
                for (int d = 0; d < DEPTH; ++d) {
                    const int i = i0 + d;
                    if (i < n_kb && ok) {
                        const int s = i % STAGES;
                        if (i >= STAGES) {
                            ok = mbar_wait(&empty_bar[s], ((i / STAGES) - 1) & 1);
                            if (!ok) atomicExch(&failed, 1);
                        }
                        if (ok) {
                            unsigned char* b = tiles + (size_t)s * STAGE_BYTES + A_BYTES;
#pragma unroll
                            for (int j = 0; j < CHUNKS; ++j) {
                                const int t = (te + j * 128) / 8;          // row of the tile
                                float o[8];
#pragma unroll
                                for (int q = 0; q < 8; ++q) o[q] = v[d][j][q] * rstd[j] * g[d][q];
                                store8(reinterpret_cast<__nv_bfloat16*>(b + t * 128 + ((c8 ^ (t & 7)) << 4)), o);
                            }
                            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                            __syncwarp();
                            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(&full_bar[s])) : "memory");
                        }
                    }
                    fetch(i + DEPTH, d);
                }
            }
        }
        {
            const int S = p.splits, rows_per = TC_BM >> p.log_splits, half = rows_per >> 1;
            const int rl = te & (rows_per - 1);
            const int row = p.mode == GF_SWIGLU ? (rl < half ? split * half + rl : 64 + split * half + (rl - half)) : split * rows_per + rl;
            const int n = tile_m * TC_BM + row;
            if (!ROPE && p.bias && n < p.n_out) pre_bias = p.bias[n];
            if constexpr (ROPE) {
                const int n_lo = tile_m * TC_BM + row_of_pair(split * half + (te & (half - 1)), p.pair_log);
                const int t = tile_n * BN + (te >> (6 - p.log_splits));
                if (n_lo < p.n_out && t < p.T) {
                    const int dist = 1 << p.pair_log, h = n_lo >> (p.pair_log + 1);
                    if (p.bias) { pre_x[0] = p.bias[n_lo]; pre_x[1] = p.bias[n_lo + dist]; }
                    if (h < r.nh + r.nkv) {
                        const float2 f = r.cos_sin[(size_t)t * dist + (n_lo & (dist - 1))];
                        pre_x[2] = f.x; pre_x[3] = f.y;
                    }
                    if (h >= r.nh) {
                        const int pos = r.positions[t];
                        pre_page = r.block_table[(size_t)r.row_req[t] * r.max_pages + pos / r.page_size];
                        pre_slot = pos % r.page_size;
                    }
                }
            }
            if (!ROPE && p.mode == GF_RESIDUAL && n < p.n_out) {
                const int t_real = min(BN, p.T - tile_n * BN);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int c = (te >> (7 - p.log_splits)) + i * S;
                    if (c < t_real) pre_x[i] = ((const float*)p.out)[(size_t)(tile_n * BN + c) * p.ldo + n];
                }
            }
        }
        if (ok && n_kb > 0) {
            ok = mbar_wait(&acc_bar, 0);
            if (!ok) atomicExch(&failed, 1);
            tc_fence_after();
        }
        // Row m of this CTA's accumulator goes to the rank that owns it, into that rank's recv[my rank][token][row
        // of its share].  (swiglu: a rank owns rows of the gate and the rows of up that belong to them.)
        const int S = p.splits, rank = split;
        const int rows_per = TC_BM >> p.log_splits, half = rows_per >> 1;  // powers of two
        const int m_local = quarter * 32 + lane;
        int owner, rl;
        if constexpr (ROPE) {
            const int j = pair_of_row(m_local, p.pair_log);
            owner = j >> (6 - p.log_splits); rl = side_of_row(m_local, p.pair_log) * half + (j & (half - 1));
        } else if (p.mode == GF_SWIGLU) {
            const int m = m_local & 63;
            owner = m >> (6 - p.log_splits); rl = (m_local >> 6) * half + (m & (half - 1));
        } else {
            owner = m_local >> (7 - p.log_splits); rl = m_local & (rows_per - 1);
        }
        const int t_real = min(BN, p.T - tile_n * BN);                     // columns beyond it are padding
        if (S > 1) cluster_wait();                                         // the peers run (first use of the barrier)
        // where token 0 of this row goes: the owner's recv[rank][0][rl] (one token further is rows_per floats on)
        const unsigned dst0 = peer_addr(smem_u32(recv) + (unsigned)(rank * BN * rows_per + rl) * 4u, (unsigned)owner);
#pragma unroll 1
        for (int c = 0; c < BN && c < t_real; c += 16) {
            unsigned r[16];
            if (ok && n_kb > 0) {
                tc_ld16(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)c, r);
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) r[j] = 0u;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                if (c + j < t_real) st_cluster(dst0 + (unsigned)((c + j) * rows_per) * 4u, __uint_as_float(r[j]));
            }
        }
        tc_fence_before();
    }
    if (p.splits > 1) {
        if (warp < 2) cluster_wait();                                      // (these warps' half of the first use)
        cluster_sync_all();                                                // second: every rank has what the others sent it
    } else {
        __syncthreads();
    }

    if (warp >= 2) {
        const int te = threadIdx.x - 64;
        const int S = p.splits, rank = split;
        const int rows_per = TC_BM >> p.log_splits, half = rows_per >> 1;
        const int t_real = min(BN, p.T - tile_n * BN);
        // thread te: row te % rows_per of this rank's share, tokens te / rows_per, + S, + 2 S, ...
        const int rl = te & (rows_per - 1);
        const int row = p.mode == GF_SWIGLU ? (rl < half ? rank * half + rl : 64 + rank * half + (rl - half)) : rank * rows_per + rl;
        const int n = tile_m * TC_BM + row;
        const float bias = pre_bias;
        const int c0 = te >> (7 - p.log_splits);
        const int part = BN * rows_per;                                    // floats between two ranks' parts
        // the sum over the ranks, in rank order (the loads go out together; S is 1, 2, 4, 8 or 16)
        auto total = [&](int c) { return ranks_sum(recv + c * rows_per + rl, part, S) + bias; };
        if constexpr (ROPE) {
            // a thread adds up feature d of a head and feature d + hd / 2 over the ranks, rotates the pair (queries and
            // keys) and writes both: a query into q, a key or a value into its token's page and slot of the cache
            const int i = te & (half - 1);
            const int dist = 1 << p.pair_log, hd = dist << 1;
            const int n_lo = tile_m * TC_BM + row_of_pair(rank * half + i, p.pair_log);
            const int h = n_lo >> (p.pair_log + 1), d = n_lo & (dist - 1);
            const int c_first = te >> (6 - p.log_splits);
            if (n_lo < p.n_out) {
                for (int c = c_first; c < t_real; c += 2 << p.log_splits) {
                    const int t = tile_n * BN + c;
                    float lo = ranks_sum(recv + c * rows_per + i, part, S) + pre_x[0];
                    float hi = ranks_sum(recv + c * rows_per + half + i, part, S) + pre_x[1];
                    if (h < r.nh + r.nkv) {
                        const float2 f = c == c_first ? make_float2(pre_x[2], pre_x[3]) : r.cos_sin[(size_t)t * dist + d];
                        const float cross_lo = __fmul_rn(hi, f.y), cross_hi = __fmul_rn(lo, f.y);
                        const float r_lo = __fmaf_rn(lo, f.x, -cross_lo), r_hi = __fmaf_rn(hi, f.x, cross_hi);
                        lo = r_lo; hi = r_hi;
                    }
                    __nv_bfloat16* dst;
                    if (h < r.nh) {
                        dst = (__nv_bfloat16*)p.out + (size_t)t * p.ldo + (size_t)h * hd + d;
                    } else {
                        int page = pre_page, slot = pre_slot;
                        if (c != c_first) {
                            const int pos = r.positions[t];
                            page = r.block_table[(size_t)r.row_req[t] * r.max_pages + pos / r.page_size];
                            slot = pos % r.page_size;
                        }
                        if (page < 0 || page >= r.num_pages) {
                            if (p.status) atomicOr(p.status, BG_STATUS_BAD_PAGE);
                            continue;
                        }
                        const bool is_v = h >= r.nh + r.nkv;
                        const int kvh = is_v ? h - r.nh - r.nkv : h - r.nh;
                        dst = r.kv_pool + (((size_t)page * 2 + (is_v ? 1 : 0)) * r.nkv + kvh) * ((size_t)r.page_size * hd) +
                              (size_t)slot * hd + d;
                    }
                    dst[0] = __float2bfloat16_rn(lo);
                    dst[dist] = __float2bfloat16_rn(hi);
                }
            }
        } else if (p.mode == GF_PLAIN) {
            if (n < p.n_out) {
                if (p.out_dtype == BG_DTYPE_F32) {
                    float* po = (float*)p.out + (size_t)(tile_n * BN + c0) * p.ldo + n;
#pragma unroll 4
                    for (int c = c0; c < t_real; c += S, po += (size_t)S * p.ldo) *po = total(c);
                } else {
                    __nv_bfloat16* po = (__nv_bfloat16*)p.out + (size_t)(tile_n * BN + c0) * p.ldo + n;
#pragma unroll 4
                    for (int c = c0; c < t_real; c += S, po += (size_t)S * p.ldo) *po = __float2bfloat16_rn(total(c));
                }
            }
        } else if (p.mode == GF_RESIDUAL) {
            // x += product; the squares of a token's new values over this rank's rows are added up by the lanes that
            // hold them (shuffles, when a rank's rows fit a warp: four ranks and more) or through shared memory
            const bool by_lanes = rows_per <= 32;
            float* po = (float*)p.out + (size_t)(tile_n * BN + c0) * p.ldo + n;
            auto leave = [&](int c, bool have, float x) {
                float v = x * x;
                if (by_lanes) {
                    for (int m = rows_per >> 1; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
                    if (rl == 0 && have && p.ssq_out)
                        p.ssq_out[(size_t)(tile_m * S + rank) * p.ssq_out_stride + tile_n * BN + c] = v;
                } else if (have) {
                    sq[c * rows_per + rl] = v;
                }
            };
#pragma unroll
            for (int i = 0; i < 4; ++i) {                                  // the values asked for ahead
                const int c = c0 + i * S;
                const bool have = c < t_real;
                if (by_lanes ? __any_sync(0xffffffffu, have) != 0 : have) {
                    float x = 0.0f;
                    if (have && n < p.n_out) {
                        x = pre_x[i] + total(c);
                        po[(size_t)i * S * p.ldo] = x;
                    }
                    leave(c, have, x);
                }
            }
            po += (size_t)4 * S * p.ldo;
            for (int c = c0 + 4 * S;; c += S, po += (size_t)S * p.ldo) {
                const bool have = c < t_real;
                if (!(by_lanes ? __any_sync(0xffffffffu, have) != 0 : have)) break;
                float x = 0.0f;
                if (have && n < p.n_out) {
                    x = *po + total(c);
                    *po = x;
                }
                leave(c, have, x);
            }
            if (!by_lanes) {
                epilogue_sync();
                // the sum of squares of this rank's rows, token by token, in row order
                if (te < t_real) {
                    float acc = 0.0f;
                    for (int i = 0; i < rows_per; ++i) acc += sq[te * rows_per + i];
                    if (p.ssq_out) p.ssq_out[(size_t)(tile_m * S + rank) * p.ssq_out_stride + tile_n * BN + te] = acc;
                }
            }
        } else {
            // SwiGLU: a thread adds up a gate value and its up value over the ranks and writes the result
            const int i = te & (half - 1);
            const int n_gate = tile_m * TC_BM + rank * half + i;           // the gate's row of the weight; its up row is 64 on
            const float bias_g = p.bias ? p.bias[n_gate] : 0.0f, bias_u = p.bias ? p.bias[n_gate + 64] : 0.0f;
            for (int c = te >> (6 - p.log_splits); c < t_real; c += 2 << p.log_splits) {
                const float g = ranks_sum(recv + c * rows_per + i, part, S) + bias_g;
                const float u = ranks_sum(recv + c * rows_per + half + i, part, S) + bias_u;
                ((__nv_bfloat16*)p.out)[(size_t)(tile_n * BN + c) * p.ldo + tile_m * 64 + rank * half + i] =
                    __float2bfloat16_rn(__fdividef(g, 1.0f + __expf(-g)) * u);   // as the SwiGLU kernel does for a bfloat16 result
            }
        }
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && failed && p.status) atomicOr(p.status, BG_STATUS_TIMEOUT);
}

template <int BN, int STAGES, bool ROPE>
static int gf_launch_stages(const CUtensorMap& mw, const CUtensorMap& mx, const FusedParams& p, const RopeParams* rope,
                            cudaStream_t stream) {
    auto kern = gemm_fused_kernel<BN, STAGES, ROPE>;
    size_t smem = (size_t)STAGES * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + (size_t)BN * TC_BM * 4 + 1024;
    static bool set = false;
    if (!set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);    // clusters of 16
        if (e != cudaSuccess) return (int)e;
        set = true;
    }
    dim3 grid((p.n_out + TC_BM - 1) / TC_BM, (p.T + BN - 1) / BN, p.splits);
    cudaError_t e;
    if constexpr (ROPE) e = launch_cluster(kern, grid, dim3(TC_THREADS), smem, stream, p.splits, mw, mx, p, *rope);
    else e = launch_cluster(kern, grid, dim3(TC_THREADS), smem, stream, p.splits, mw, mx, p, NoRope());
    if (e != cudaSuccess) return (int)e;
    BG_LAUNCH_CHECK();
    return BG_OK;
}

// A grid that leaves SMs to spare has a CTA alone on its SM: eight stages then keep enough bytes on their way
// from HBM (the stream of a few CTAs is bound by what they have in flight); else four, so that two CTAs share an SM.
template <int BN>
static int gf_launch(const CUtensorMap& mw, const CUtensorMap& mx, const FusedParams& p, const RopeParams* rope,
                     cudaStream_t stream) {
    const long long ctas = (long long)((p.n_out + TC_BM - 1) / TC_BM) * ((p.T + BN - 1) / BN) * p.splits;
    if (p.mode == GF_ROPE) {
        if (BN <= 32 && ctas <= sm_count() && p.kb_per_split > 4) return gf_launch_stages<BN, 8, true>(mw, mx, p, rope, stream);
        return gf_launch_stages<BN, 4, true>(mw, mx, p, rope, stream);
    }
    if (BN <= 32 && ctas <= sm_count() && p.kb_per_split > 4) return gf_launch_stages<BN, 8, false>(mw, mx, p, rope, stream);
    return gf_launch_stages<BN, 4, false>(mw, mx, p, rope, stream);
}

}  // namespace bg

using namespace bg;

struct RopeArgs {
    const float* cos_sin;
    const int *positions, *row_req, *block_table;
    void* kv_pool;
    int max_pages, num_pages, page_size, nh, nkv, hd;
};

static int gemm_fused_run(const void* W, int n_out, int K, int ldw, const void* X, int ldx, const float* xf, int ldxf,
                          const float* ssq_in, int n_ssq_in, int ssq_in_stride, const void* norm_w, float eps, int T,
                          const float* bias, int mode, void* out, int out_dtype, int ldo, float* ssq_out,
                          int ssq_out_stride, int splits, const RopeArgs* rope, unsigned* status, cudaStream_t stream) {
    if (T <= 0 || n_out <= 0) return BG_OK;
    if (K <= 0 || T > 64) return BG_ERR_SHAPE;
    if (splits != 1 && splits != 2 && splits != 4 && splits != 8 && splits != 16) return BG_ERR_SHAPE;
    if ((ldw % 8) || (K % 8) || ((uintptr_t)W % 16)) return BG_ERR_ALIGN;
    if ((X == nullptr) == (xf == nullptr)) return BG_ERR_SHAPE;
    if (X && ((ldx % 8) || ((uintptr_t)X % 16))) return BG_ERR_ALIGN;
    if (xf && ((ldxf % 4) || ((uintptr_t)xf % 16) || ((uintptr_t)norm_w % 16) || !ssq_in || !norm_w || n_ssq_in < 1)) return BG_ERR_ALIGN;
    FusedParams p;
    RopeParams rp;
    memset(&p, 0, sizeof(p));
    memset(&rp, 0, sizeof(rp));
    if (mode == GF_PLAIN) {
        if (out_dtype != BG_DTYPE_F32 && out_dtype != BG_DTYPE_BF16) return BG_ERR_DTYPE;
    } else if (mode == GF_RESIDUAL) {
        if (out_dtype != BG_DTYPE_F32) return BG_ERR_DTYPE;
    } else if (mode == GF_SWIGLU) {
        if (out_dtype != BG_DTYPE_BF16) return BG_ERR_DTYPE;
        if (n_out % TC_BM) return BG_ERR_SHAPE;
        p.pair_log = 6;
    } else if (mode == GF_ROPE) {
        if (!rope || out_dtype != BG_DTYPE_BF16) return BG_ERR_DTYPE;
        // whole heads in a tile, so that a feature and its partner meet in one CTA
        if (rope->hd != 32 && rope->hd != 64 && rope->hd != 128) return BG_ERR_UNSUPPORTED;
        if (rope->nh < 1 || rope->nkv < 1 || n_out != (rope->nh + 2 * rope->nkv) * rope->hd) return BG_ERR_SHAPE;
        if (!rope->cos_sin || !rope->positions || !rope->row_req || !rope->block_table || !rope->kv_pool) return BG_ERR_SHAPE;
        if (rope->page_size < 1 || rope->max_pages < 1 || rope->num_pages < 1 || ((uintptr_t)rope->cos_sin % 8)) return BG_ERR_SHAPE;
        p.pair_log = rope->hd == 32 ? 4 : rope->hd == 64 ? 5 : 6;
        rp.cos_sin = (const float2*)rope->cos_sin; rp.positions = rope->positions; rp.row_req = rope->row_req;
        rp.block_table = rope->block_table; rp.kv_pool = (__nv_bfloat16*)rope->kv_pool; rp.max_pages = rope->max_pages;
        rp.num_pages = rope->num_pages; rp.page_size = rope->page_size; rp.nh = rope->nh; rp.nkv = rope->nkv;
    } else {
        return BG_ERR_SHAPE;
    }
    const int n_kb = (K + TC_BK - 1) / TC_BK;
    p.xf = xf; p.ldxf = ldxf; p.ssq_in = ssq_in; p.n_ssq_in = n_ssq_in; p.ssq_in_stride = ssq_in_stride;
    p.norm_w = (const __nv_bfloat16*)norm_w; p.eps = eps;
    p.bias = bias; p.mode = mode; p.out = out; p.out_dtype = out_dtype; p.ldo = ldo;
    p.ssq_out = ssq_out; p.ssq_out_stride = ssq_out_stride;
    p.n_out = n_out; p.T = T; p.K = K; p.splits = splits;
    p.kb_per_split = (n_kb + splits - 1) / splits;
    p.log_splits = 0;
    while ((1 << p.log_splits) < splits) ++p.log_splits;
    p.status = status;
    if ((long long)(splits - 1) * p.kb_per_split >= n_kb) return BG_ERR_SHAPE;      // an empty range of K
    const int bn = T <= 16 ? 16 : T <= 32 ? 32 : 64;
    CUtensorMap mw, mx;
    int rc = weight_map(&mw, W, n_out, K, ldw);
    if (rc != BG_OK) return rc;
    if (X) {
        rc = make_map(&mx, X, T, K, ldx, bn);
        if (rc != BG_OK) return rc;
    } else {
        memset(&mx, 0, sizeof(mx));
    }
    switch (bn) {
        case 16: return gf_launch<16>(mw, mx, p, &rp, stream);
        case 32: return gf_launch<32>(mw, mx, p, &rp, stream);
        default: return gf_launch<64>(mw, mx, p, &rp, stream);
    }
}

// See the head of the file.  X (bfloat16 [T, K], row stride ldx) or xf (float [T, K], row stride ldxf, with
// ssq_in, norm_w and eps) is the left operand; splits is 1, 2, 4, 8 or 16.
extern "C" int bg_gemm_fused(const void* W, int n_out, int K, int ldw, const void* X, int ldx, const float* xf, int ldxf,
                             const float* ssq_in, int n_ssq_in, int ssq_in_stride, const void* norm_w, float eps, int T,
                             const float* bias, int mode, void* out, int out_dtype, int ldo, float* ssq_out,
                             int ssq_out_stride, int splits, unsigned* status, cudaStream_t stream) {
    if (mode == GF_ROPE) return BG_ERR_SHAPE;
    return gemm_fused_run(W, n_out, K, ldw, X, ldx, xf, ldxf, ssq_in, n_ssq_in, ssq_in_stride, norm_w, eps, T, bias, mode,
                          out, out_dtype, ldo, ssq_out, ssq_out_stride, splits, nullptr, status, stream);
}

// The q/k/v product of a step of few tokens with rotation and cache append behind it: W [(nh + 2 nkv) hd, K], the
// left operand as above; q_out bfloat16 [T][q_stride]; cos_sin [T][hd / 2][2]; the pool of the layer
// [num_pages][2][nkv][page_size][hd] bfloat16.  Head sizes other than 32, 64 and 128 are refused
// (BG_ERR_UNSUPPORTED): the caller then runs the product and the rotation as two kernels.
extern "C" int bg_gemm_fused_rope(const void* W, int K, int ldw, const void* X, int ldx, const float* xf, int ldxf,
                                  const float* ssq_in, int n_ssq_in, int ssq_in_stride, const void* norm_w, float eps, int T,
                                  const float* bias, void* q_out, int q_stride, const float* cos_sin, const int* positions,
                                  const int* row_req, const int* block_table, int max_pages, void* kv_pool, int num_pages,
                                  int page_size, int nh, int nkv, int hd, int splits, unsigned* status, cudaStream_t stream) {
    RopeArgs r;
    r.cos_sin = cos_sin; r.positions = positions; r.row_req = row_req; r.block_table = block_table; r.kv_pool = kv_pool;
    r.max_pages = max_pages; r.num_pages = num_pages; r.page_size = page_size; r.nh = nh; r.nkv = nkv; r.hd = hd;
    if (nh < 1 || nkv < 1 || hd < 1) return BG_ERR_SHAPE;
    return gemm_fused_run(W, (nh + 2 * nkv) * hd, K, ldw, X, ldx, xf, ldxf, ssq_in, n_ssq_in, ssq_in_stride, norm_w, eps, T,
                          bias, GF_ROPE, q_out, BG_DTYPE_BF16, q_stride, nullptr, 0, splits, &r, status, stream);
}
