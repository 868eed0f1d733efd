// out[t, n] = sum_k X[t, k] * W[n, k] for steps of many tokens (prompt portions), on the fifth-generation tensor
// cores with PAIRS of CTAs: a persistent kernel, one pair (a thread block cluster of two, on the two SMs of a
// TPC) per tile of 256 tokens x 256 (or 192, or 128) output features.
//
//   tokens are the M side here and the weights the N side (the reverse of gemm_tcgen05.cu, which streams the
//   weights once for a handful of tokens): a thread of the epilogue then owns a token's row of consecutive
//   features, so SwiGLU (gate and up features interleaved in blocks of 64 rows of the weight) is a thread's own
//   business, and rows go out as whole 128-byte lines.
//   One thread of the pair's first CTA issues tcgen05.mma.cta_group::2 (M = 256, N = the tile's width): each CTA
//   brings its own 128 tokens and HALF of the tile's weight rows into its shared memory (32 KB a stage instead of 48
//   for 256 features), the instruction reads both halves, and each CTA's tensor memory receives the accumulator of
//   its own 128 tokens.  That halving of the operand traffic per flop is what lets the tensor pipe run near its
//   peak: an SM fetches its operands at 64 bytes a cycle, which is just what a tile of 256 x 256 needs.
//   The accumulator is double-buffered in tensor memory (two buffers of the tile's width): the four epilogue warps
//   of each CTA drain tile i (tcgen05.ld, convert, stage in shared memory, TMA store or TMA reduction) while the
//   MMAs of tile i + 1 run.
//   Epilogues: plain (+ bias) as bfloat16; SwiGLU; or added into the float residual stream by
//   cp.reduce.async.bulk.tensor ... add, so that the SM never reads the stream.
//
// Barriers (mbarriers; a wait is bounded and records BG_STATUS_TIMEOUT):
//   full[s]       in the first CTA: one arrival (its producer's expect_tx of BOTH CTAs' bytes) + the bytes; the second
//                 CTA's copies complete on the first CTA's barrier (cp.async.bulk.tensor with .cta_group::2)
//   empty[s]      in both CTAs: tcgen05.commit (multicast to the pair) when the stage's MMAs have read it
//   acc_full[b]   in both CTAs: tcgen05.commit (multicast) after a tile's last MMA
//   acc_empty[b]  in the first CTA: 8 arrivals, one per epilogue warp of the pair, when the warp has read buffer b
// No copy here is a multicast copy: each CTA fetches its own operands.
#include "tc_common.cuh"

namespace bg {

constexpr int GP_BM = 128;                 // tokens per CTA (256 per pair)
constexpr int GP_THREADS = 192;            // warp 0: TMA, warp 1: MMA + tensor memory, warps 2-5: epilogue
constexpr unsigned GP_A_BYTES = GP_BM * TC_BK * 2;
constexpr unsigned GP_OUT_BYTES = GP_BM * 128;                        // a staging buffer: 128 rows of 64 bfloat16
constexpr int GP_MODE_PLAIN = 0;           // out[t, n] (+ bias[n]) as bfloat16
constexpr int GP_MODE_SWIGLU = 1;          // out[t, j] = silu(gate) * up, the weight's rows interleaved in blocks of 64
constexpr int GP_MODE_RESIDUAL = 2;        // out (float, the residual stream) [t, n] += product (+ bias[n])
// A tile is 256 tokens x BN output features, BN = 256, 192 or 128: a CTA loads BN / 2 rows of the weight.  The widest
// tile that keeps the pairs of the device busy is chosen on the host: a narrow matrix has too few tiles of 256.
template <int BN> struct GpTile {
    static constexpr unsigned B_BYTES = (BN / 2) * TC_BK * 2;
    static constexpr unsigned STAGE_BYTES = GP_A_BYTES + B_BYTES;             // 32, 28 or 24 KB
    static constexpr unsigned TMEM_COLS = BN <= 128 ? 256 : 512;              // two accumulators of BN columns
};

struct PairParams {
    const float* bias;      // [n_out] or null
    int n_out, T, K;
    int tiles_m, tiles_n;   // tiles of 256 tokens and of BN features
    unsigned* status;
};

__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// A TMA load whose completion is counted on a barrier of the pair's first CTA.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y, unsigned bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tc_commit_pair(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
                 ::"r"(smem_u32(bar)), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc, unsigned idesc,
                                            unsigned accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(unsigned bar_cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
// 16 bytes into a staging buffer of 128 rows x 128 bytes in the 128-byte swizzle of the store's tensor map
__device__ __forceinline__ void stage_store16(unsigned char* buf, int row, int chunk, uint4 v) {
    *reinterpret_cast<uint4*>(buf + row * 128 + ((chunk ^ (row & 7)) << 4)) = v;
}

template <int STAGES, int MODE, int BN>
__global__ void __launch_bounds__(GP_THREADS)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                 const __grid_constant__ CUtensorMap map_out, PairParams p) {
    extern __shared__ unsigned char gp_smem_raw[];
    constexpr unsigned GP_STAGE_BYTES = GpTile<BN>::STAGE_BYTES;
    constexpr int GP_HALF_N = BN / 2;
    constexpr int GP_BN = BN;
    unsigned char* tiles = (unsigned char*)(((uintptr_t)gp_smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* staging = tiles + (size_t)STAGES * GP_STAGE_BYTES;
    __shared__ __align__(8) unsigned long long full_bar[STAGES];
    __shared__ __align__(8) unsigned long long empty_bar[STAGES];
    __shared__ __align__(8) unsigned long long acc_full[2];
    __shared__ __align__(8) unsigned long long acc_empty[2];
    __shared__ unsigned tmem_base_sh;
    __shared__ int failed;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = cluster_rank();
    const int n_pairs = gridDim.x >> 1, pair = blockIdx.x >> 1;
    const int n_tiles = p.tiles_m * p.tiles_n;
    const int n_kb = (p.K + TC_BK - 1) / TC_BK;

    pdl_launch();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(&tmem_base_sh)), "r"(GpTile<BN>::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                     // the peer's barriers are initialised before anything is signalled there
    tc_fence_after();
    const unsigned tmem_base = tmem_base_sh;

    if (warp == 0) {
        // ---------------- TMA producer (in both CTAs: own tokens, own half of the weight rows)
        if (lane == 0) {
            pdl_wait();
            int it = 0;
            bool ok = true;
            for (int tile = pair; tile < n_tiles && ok; tile += n_pairs) {
                const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
                const int row_x = tm * (2 * GP_BM) + (int)rank * GP_BM;
                const int row_w = tn * GP_BN + (int)rank * GP_HALF_N;
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait(&empty_bar[s], ((it / STAGES) - 1) & 1)) { ok = false; break; }
                    unsigned char* a = tiles + (size_t)s * GP_STAGE_BYTES;
                    if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * GP_STAGE_BYTES);
                    const unsigned bar = peer_addr(smem_u32(&full_bar[s]), 0);
                    tma_load_2d_pair(a, &map_x, kb * TC_BK, row_x, bar);
                    tma_load_2d_pair(a + GP_A_BYTES, &map_w, kb * TC_BK, row_w, bar);
                }
            }
            if (!ok) atomicExch(&failed, 1);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: one thread of the pair's first CTA
        if (lane == 0 && rank == 0) {
            constexpr unsigned idesc = instr_desc_bf16(2 * GP_BM, GP_BN);
            int it = 0, t_idx = 0;
            bool ok = true;
            for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++t_idx) {
                const int b = t_idx & 1;
                if (t_idx >= 2 && !mbar_wait(&acc_empty[b], ((t_idx >> 1) - 1) & 1)) { ok = false; break; }
                tc_fence_after();
                const unsigned d = tmem_base + (unsigned)(b * GP_BN);
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&full_bar[s], (it / STAGES) & 1)) { ok = false; break; }
                    tc_fence_after();
                    const unsigned a_addr = smem_u32(tiles + (size_t)s * GP_STAGE_BYTES);
                    const unsigned b_addr = a_addr + GP_A_BYTES;
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)
                        tc_mma_pair(d, smem_desc_sw128(a_addr + k * 32), smem_desc_sw128(b_addr + k * 32), idesc,
                                    (kb > 0 || k > 0) ? 1u : 0u);
                    tc_commit_pair(&empty_bar[s]);      // the stage is free in both CTAs once these MMAs have read it
                }
                if (ok) tc_commit_pair(&acc_full[b]);   // both CTAs' epilogues: every MMA of the tile is complete
            }
            if (!ok) atomicExch(&failed, 1);
        }
    } else {
        // ---------------- epilogue: warps 2..5 own tensor-memory lanes 32 * (warp % 4) .. + 31, a token each
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const bool elected = (warp == 2 && lane == 0);
        const unsigned acc_empty_first = peer_addr(smem_u32(&acc_empty[0]), 0);
        int t_idx = 0, q = 0;
        bool ok = true;
        pdl_wait();
        for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++t_idx) {
            const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
            const int b = t_idx & 1;
            if (!mbar_wait(&acc_full[b], (t_idx >> 1) & 1)) { ok = false; break; }
            tc_fence_after();
            const unsigned t_addr = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(b * GP_BN);
            const int row0 = tm * (2 * GP_BM) + (int)rank * GP_BM;
            if (MODE == GP_MODE_RESIDUAL) {
                // 32 features of the thread's token at a time go into the staging buffer as floats (a row of 128
                // bytes), and a TMA reduction adds the buffer to the stream in global memory: the SM never reads
                // the stream, and every element is added to exactly once
#pragma unroll 1
                for (int c = 0; c < GP_BN / 32; ++c, ++q) {
                    unsigned char* buf = staging + (size_t)(q & 1) * GP_OUT_BYTES;
                    if (elected) asm volatile("cp.async.bulk.wait_group.read 1;\n" ::: "memory");
                    asm volatile("bar.sync 1, 128;\n" ::: "memory");
                    unsigned g[32];
                    tc_ld32_nowait(t_addr + (unsigned)(c * 32), g);
                    tc_wait_ld();
                    if (c == GP_BN / 32 - 1) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(acc_empty_first + (unsigned)(b * sizeof(unsigned long long)));
                    }
                    const int n0 = tn * GP_BN + c * 32;
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        float o[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            o[j] = __uint_as_float(g[4 * v + j]) + ((p.bias && n0 + 4 * v + j < p.n_out) ? __ldg(p.bias + n0 + 4 * v + j) : 0.0f);
                        stage_store16(buf, row, v, make_uint4(__float_as_uint(o[0]), __float_as_uint(o[1]), __float_as_uint(o[2]),
                                                              __float_as_uint(o[3])));
                    }
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                    asm volatile("bar.sync 1, 128;\n" ::: "memory");
                    if (elected) {
                        tma_reduce_add_2d(&map_out, buf, n0, row0);
                        asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
                    }
                }
                continue;
            }
            constexpr int CHUNKS = MODE == GP_MODE_SWIGLU ? GP_BN / 128 : GP_BN / 64;
#pragma unroll 1
            for (int c = 0; c < CHUNKS; ++c, ++q) {
                unsigned char* buf = staging + (size_t)(q & 1) * GP_OUT_BYTES;
                if (elected) asm volatile("cp.async.bulk.wait_group.read 1;\n" ::: "memory");
                asm volatile("bar.sync 1, 128;\n" ::: "memory");     // the store that read this buffer two chunks ago is done
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    unsigned g[32], u[32];
                    float o[32];
                    if (MODE == GP_MODE_SWIGLU) {
                        tc_ld32_nowait(t_addr + (unsigned)(c * 128 + h * 32), g);
                        tc_ld32_nowait(t_addr + (unsigned)(c * 128 + 64 + h * 32), u);
                        tc_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const float gv = __uint_as_float(g[j]), uv = __uint_as_float(u[j]);
                            o[j] = __fdividef(gv, 1.0f + __expf(-gv)) * uv;
                        }
                    } else {
                        tc_ld32_nowait(t_addr + (unsigned)(c * 64 + h * 32), g);
                        tc_wait_ld();
                        const int n0 = tn * GP_BN + c * 64 + h * 32;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            o[j] = __uint_as_float(g[j]) + ((p.bias && n0 + j < p.n_out) ? __ldg(p.bias + n0 + j) : 0.0f);
                    }
                    if (c == CHUNKS - 1 && h == 1) {
                        // the buffer of tensor memory has been read: the MMAs of the tile after next may overwrite it
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(acc_empty_first + (unsigned)(b * sizeof(unsigned long long)));
                    }
#pragma unroll
                    for (int v = 0; v < 4; ++v)
                        stage_store16(buf, row, h * 4 + v,
                                      make_uint4(pack_bf16(o[8 * v], o[8 * v + 1]), pack_bf16(o[8 * v + 2], o[8 * v + 3]),
                                                 pack_bf16(o[8 * v + 4], o[8 * v + 5]), pack_bf16(o[8 * v + 6], o[8 * v + 7])));
                }
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                asm volatile("bar.sync 1, 128;\n" ::: "memory");
                if (elected) {
                    const int col0 = MODE == GP_MODE_SWIGLU ? tn * (GP_BN / 2) + c * 64 : tn * GP_BN + c * 64;
                    tma_store_2d(&map_out, buf, col0, row0);
                    asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
                }
            }
        }
        if (elected) asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory");
        if (!ok) atomicExch(&failed, 1);
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                     // neither CTA frees tensor memory or leaves while its peer may still signal it
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(GpTile<BN>::TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && failed && p.status) atomicOr(p.status, BG_STATUS_TIMEOUT);
}

template <int STAGES, int MODE, int BN>
static int gp_launch(const CUtensorMap& mx, const CUtensorMap& mw, const CUtensorMap& mo, const PairParams& p, cudaStream_t stream) {
    auto kern = gemm_pair_kernel<STAGES, MODE, BN>;
    const size_t smem = (size_t)STAGES * GpTile<BN>::STAGE_BYTES + 2 * GP_OUT_BYTES + 1024;
    static bool set = false;
    if (!set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        set = true;
    }
    const int n_tiles = p.tiles_m * p.tiles_n;
    int pairs = sm_count() / 2;
    if (pairs > n_tiles) pairs = n_tiles;
    if (pairs < 1) return BG_ERR_UNSUPPORTED;
    // a kernel that issues cta_group::2 instructions is launched with its pairs along x (a launch with the cluster
    // along z is refused as a misconfigured cluster)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs); cfg.blockDim = dim3(GP_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = 2; attr[n].val.clusterDim.y = 1; attr[n].val.clusterDim.z = 1;
    ++n;
    cfg.attrs = attr; cfg.numAttrs = n;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, mx, mw, mo, p);
    if (e != cudaSuccess) return (int)e;
    BG_LAUNCH_CHECK();
    return BG_OK;
}

// The tile width for a product of T rows with n_out output features: the one whose rounds of tiles over the
// device's pairs cost least.  A tile's cost is the larger of its MMA time (in proportion to its width) and the
// time its operands need to reach an SM (16 KB of tokens and 64 bytes per feature, at 64 bytes a cycle): 512, 448
// and 384 cycles per k-block for 256, 192 and 128 features.  Ties go to the wider tile.
static int gp_tile_width(int T, int n_out, int mode) {
    static int forced = [] { const char* e = getenv("BEGLIN_B200_PAIR_BN"); return e ? atoi(e) : 0; }();
    if (forced == 256 || forced == 128 || (forced == 192 && mode != GP_MODE_SWIGLU)) return forced;
    const int pairs = sm_count() / 2 > 0 ? sm_count() / 2 : 1;
    const int tiles_m = (T + 2 * GP_BM - 1) / (2 * GP_BM);
    const int widths[3] = {256, 192, 128}, cost[3] = {512, 448, 384};
    int best = 256;
    long long best_cost = -1;
    for (int i = 0; i < 3; ++i) {
        if (widths[i] == 192 && mode == GP_MODE_SWIGLU) continue;         // gate and up come in blocks of 64 + 64
        const long long tiles = (long long)tiles_m * ((n_out + widths[i] - 1) / widths[i]);
        const long long c = (tiles + pairs - 1) / pairs * cost[i];
        if (best_cost < 0 || c < best_cost) { best_cost = c; best = widths[i]; }
    }
    return best;
}

}  // namespace bg

using namespace bg;

// The product of many rows on pairs of CTAs.
//   mode 0: out[t, n] = sum_k X[t, k] W[n, k] (+ bias[n]) as bfloat16 [T, ldo];
//   mode 1: the rows of W are gate and up features interleaved in blocks of 64 (n_out = 2 * inner, a multiple of
//           128): out[t, j] = silu(gate_j) * up_j as bfloat16 [T, ldo] with n_out / 2 columns; no bias;
//   mode 2: out is the float residual stream [T, ldo]: out[t, n] += sum_k X[t, k] W[n, k] (+ bias[n]).
//   W: [n_out, K] bfloat16, row stride ldw; X: [T, K] bfloat16, row stride ldx; strides multiples of 8 elements
//   (ldo of mode 2: of 4), bases 16-byte aligned.
extern "C" int bg_gemm_pair(const void* W, int n_out, int K, int ldw, const void* X, int T, int ldx, const float* bias,
                            void* out, int ldo, int mode, unsigned* status, cudaStream_t stream) {
    if (T <= 0 || n_out <= 0) return BG_OK;
    if (K <= 0) return BG_ERR_SHAPE;
    if (mode != GP_MODE_PLAIN && mode != GP_MODE_SWIGLU && mode != GP_MODE_RESIDUAL) return BG_ERR_UNSUPPORTED;
    if ((ldw % 8) || (ldx % 8) || ((uintptr_t)W % 16) || ((uintptr_t)X % 16) || ((uintptr_t)out % 16)) return BG_ERR_ALIGN;
    if (mode == GP_MODE_RESIDUAL ? (ldo % 4) : (ldo % 8)) return BG_ERR_ALIGN;
    if (mode == GP_MODE_SWIGLU && (n_out % 128 || bias)) return BG_ERR_SHAPE;
    const int bn = gp_tile_width(T, n_out, mode);
    PairParams p;
    p.bias = bias; p.n_out = n_out; p.T = T; p.K = K; p.status = status;
    p.tiles_m = (T + 2 * GP_BM - 1) / (2 * GP_BM);
    p.tiles_n = (n_out + bn - 1) / bn;
    CUtensorMap mw, mx, mo;
    int rc = weight_map(&mw, W, n_out, K, ldw, bn / 2);
    if (rc != BG_OK) return rc;
    rc = make_map(&mx, X, T, K, ldx, GP_BM);
    if (rc != BG_OK) return rc;
    if (mode == GP_MODE_RESIDUAL) rc = make_map_f32(&mo, out, T, n_out, ldo, GP_BM);
    else rc = make_map(&mo, out, T, mode == GP_MODE_SWIGLU ? n_out / 2 : n_out, ldo, GP_BM);
    if (rc != BG_OK) return rc;
    if (mode == GP_MODE_SWIGLU)
        return bn == 256 ? gp_launch<6, GP_MODE_SWIGLU, 256>(mx, mw, mo, p, stream) : gp_launch<8, GP_MODE_SWIGLU, 128>(mx, mw, mo, p, stream);
    if (mode == GP_MODE_PLAIN)
        return bn == 256 ? gp_launch<6, GP_MODE_PLAIN, 256>(mx, mw, mo, p, stream)
             : bn == 192 ? gp_launch<6, GP_MODE_PLAIN, 192>(mx, mw, mo, p, stream) : gp_launch<8, GP_MODE_PLAIN, 128>(mx, mw, mo, p, stream);
    return bn == 256 ? gp_launch<6, GP_MODE_RESIDUAL, 256>(mx, mw, mo, p, stream)
         : bn == 192 ? gp_launch<6, GP_MODE_RESIDUAL, 192>(mx, mw, mo, p, stream) : gp_launch<8, GP_MODE_RESIDUAL, 128>(mx, mw, mo, p, stream);
}
