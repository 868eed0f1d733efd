// out[t, n] = sum_k X[t, k] * W[n, k] (+ bias[n]) for bfloat16 X and W with float accumulation, on
// the fifth-generation tensor cores: operand tiles are brought into shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle), one thread issues tcgen05.mma with the accumulator in
// tensor memory, and four warps read the accumulator back with tcgen05.ld for the epilogue.
//
// The weight matrix is the M side of the instruction (128 output features per CTA) and the tokens
// are the N side (16 to 256 per CTA), so a decoding step with a handful of tokens wastes no tensor
// work on padding and streams the weights once.  Both operands are K-major, which is the layout of
// the checkpoint's [out, in] matrices and of the activations [tokens, in].
//
// Split-K: blockIdx.z takes a contiguous range of 64-wide k-blocks and writes a float partial
// result out[z][t][n]; the kernel that consumes the result sums the partials in index order, so the
// order of the sum is fixed by the shapes and does not depend on the batch.
//
// Every wait on an mbarrier is bounded: when a wait runs out the thread records
// BG_STATUS_TIMEOUT in the status word and the CTA winds down (tensor memory is freed).
#include "tc_common.cuh"

namespace bg {

struct TcParams {
    const float* bias;      // [n_out] or null (added only by split 0)
    void* out;              // [splits][T][ldo] float partials, or [T][ldo] float / bfloat16
    long long split_stride; // elements between the partials of two splits
    int ldo;
    int out_dtype;
    int n_out, T, K;
    int kb_per_split;       // 64-wide k-blocks per split
    unsigned* status;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(TC_THREADS)
gemm_bf16_tn_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, TcParams p) {
    constexpr unsigned A_BYTES = TC_BM * TC_BK * 2;
    constexpr unsigned B_BYTES = BN * TC_BK * 2;
    constexpr unsigned STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr unsigned TMEM_COLS = BN < 32 ? 32 : BN;
    extern __shared__ unsigned char tc_smem_raw[];
    unsigned char* tiles = (unsigned char*)(((uintptr_t)tc_smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) unsigned long long full_bar[STAGES];
    __shared__ __align__(8) unsigned long long empty_bar[STAGES];
    __shared__ __align__(8) unsigned long long acc_bar;
    __shared__ unsigned tmem_base_sh;
    __shared__ int failed;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_m = blockIdx.x, tile_n = blockIdx.y, split = blockIdx.z;
    const int n_kb_total = (p.K + TC_BK - 1) / TC_BK;
    const int kb0 = split * p.kb_per_split;
    const int n_kb = min(p.kb_per_split, n_kb_total - kb0);

    pdl_launch();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
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

    if (warp == 0) {
        // ---------------- TMA producer
        if (lane == 0 && n_kb > 0) {
            // The weights do not depend on any earlier kernel of the step: the first stages' weight tiles
            // are requested at once, while the kernel that produces the activations may still be running.
            const int ahead = n_kb < STAGES ? n_kb : STAGES;
            for (int i = 0; i < ahead; ++i) {
                mbar_expect_tx(&full_bar[i], STAGE_BYTES);
                tma_load_2d(tiles + (size_t)i * STAGE_BYTES, &map_w, (kb0 + i) * TC_BK, tile_m * TC_BM, &full_bar[i]);
            }
            pdl_wait();
            for (int i = 0; i < ahead; ++i)
                tma_load_2d(tiles + (size_t)i * STAGE_BYTES + A_BYTES, &map_x, (kb0 + i) * TC_BK, tile_n * BN, &full_bar[i]);
            for (int i = ahead; i < n_kb; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(&empty_bar[s], ((i / STAGES) - 1) & 1)) { atomicExch(&failed, 1); break; }
                unsigned char* a = tiles + (size_t)s * STAGE_BYTES;
                unsigned char* b = a + A_BYTES;
                mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                tma_load_2d(a, &map_w, (kb0 + i) * TC_BK, tile_m * TC_BM, &full_bar[s]);
                tma_load_2d(b, &map_x, (kb0 + i) * TC_BK, tile_n * BN, &full_bar[s]);
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
                for (int k = 0; k < TC_BK / 16; ++k) {
                    tc_mma(tmem_base, smem_desc_sw128(a_addr + k * 32), smem_desc_sw128(b_addr + k * 32), idesc,
                           (i > 0 || k > 0) ? 1u : 0u);
                }
                tc_commit(&empty_bar[s]);          // the stage is free once these MMAs have read it
            }
            tc_commit(&acc_bar);                    // arrives when every MMA above is complete
        }
    } else {
        // ---------------- epilogue: warps 2..5 own tensor-memory lanes 32*(warp%4) .. +31
        const int quarter = warp & 3;
        const int m = tile_m * TC_BM + quarter * 32 + lane;
        bool ok = true;
        pdl_wait();
        if (n_kb > 0) {
            ok = mbar_wait(&acc_bar, 0);
            if (!ok) atomicExch(&failed, 1);
            tc_fence_after();
        }
        if (ok) {
            const float bias = (p.bias && split == 0 && m < p.n_out) ? p.bias[m] : 0.0f;
            const int t0 = tile_n * BN;
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                if (t0 + c >= p.T) break;                                  // warp-uniform
                unsigned r[16];
                if (n_kb > 0) {
                    tc_ld16(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)c, r);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) r[j] = 0u;
                }
                if (m < p.n_out) {
                    if (p.out_dtype == BG_DTYPE_F32) {
                        float* o = (float*)p.out + (size_t)split * p.split_stride + (size_t)(t0 + c) * p.ldo + m;
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (t0 + c + j < p.T) o[(size_t)j * p.ldo] = __uint_as_float(r[j]) + bias;
                    } else {
                        __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)(t0 + c) * p.ldo + m;
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (t0 + c + j < p.T) o[(size_t)j * p.ldo] = __float2bfloat16_rn(__uint_as_float(r[j]) + bias);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && failed && p.status) atomicOr(p.status, BG_STATUS_TIMEOUT);
}

template <int BN, int STAGES>
static int tc_launch(const CUtensorMap& mw, const CUtensorMap& mx, const TcParams& p, int splits, cudaStream_t stream) {
    auto kern = gemm_bf16_tn_tcgen05_kernel<BN, STAGES>;
    size_t smem = (size_t)STAGES * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + 1024;
    static bool set = false;
    if (!set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        set = true;
    }
    dim3 grid((p.n_out + TC_BM - 1) / TC_BM, (p.T + BN - 1) / BN, splits);
    launch(kern, grid, dim3(TC_THREADS), smem, stream, mw, mx, p);
    BG_LAUNCH_CHECK();
    return BG_OK;
}

}  // namespace bg

using namespace bg;

// out[t, n] = sum_k X[t, k] W[n, k] (+ bias[n]).
//   W: [n_out, K] bfloat16, row stride ldw; X: [T, K] bfloat16, row stride ldx (strides multiples of 8).
//   splits == 1: out is [T, ldo] in out_dtype (float or bfloat16).
//   splits  > 1: out is float [splits, T, ldo]; the caller sums over the first index.  bias goes
//                into split 0.
extern "C" int bg_gemm_bf16_tn(const void* W, int n_out, int K, int ldw, const void* X, int T, int ldx, const float* bias,
                               void* out, int out_dtype, int ldo, int splits, unsigned* status, cudaStream_t stream) {
    if (T <= 0 || n_out <= 0) return BG_OK;
    if (K <= 0 || splits < 1) return BG_ERR_SHAPE;
    if ((ldw % 8) || (ldx % 8) || ((uintptr_t)W % 16) || ((uintptr_t)X % 16)) return BG_ERR_ALIGN;
    if (splits > 1 && out_dtype != BG_DTYPE_F32) return BG_ERR_DTYPE;
    if (out_dtype != BG_DTYPE_F32 && out_dtype != BG_DTYPE_BF16) return BG_ERR_DTYPE;
    const int n_kb = (K + TC_BK - 1) / TC_BK;
    if (splits > n_kb) splits = n_kb;
    TcParams p;
    p.bias = bias; p.out = out; p.ldo = ldo; p.out_dtype = out_dtype; p.n_out = n_out; p.T = T; p.K = K;
    p.kb_per_split = (n_kb + splits - 1) / splits;
    p.split_stride = (long long)T * ldo;
    p.status = status;
    if ((long long)(splits - 1) * p.kb_per_split >= n_kb) return BG_ERR_SHAPE;      // an empty split
    const int bn = T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : T <= 128 ? 128 : 256;

    // the weight's map is made once per (pointer, shape); the activation's for every call
    CUtensorMap mw, mx;
    {
        int rc = weight_map(&mw, W, n_out, K, ldw);
        if (rc != BG_OK) return rc;
    }
    int rc = make_map(&mx, X, T, K, ldx, bn);
    if (rc != BG_OK) return rc;
    switch (bn) {
        // few tokens: the product is bound by the weight stream; four stages let three CTAs share an SM, so
        // one CTA's start and epilogue overlap the others' loads
        case 16: return tc_launch<16, 4>(mw, mx, p, splits, stream);
        case 32: return tc_launch<32, 4>(mw, mx, p, splits, stream);
        case 64: return tc_launch<64, 4>(mw, mx, p, splits, stream);
        case 128: return tc_launch<128, 3>(mw, mx, p, splits, stream);
        default: {
            // many tokens: the product is bound by the tensor cores.  With more CTAs than SMs, two stages keep
            // a CTA under half of an SM's shared memory, so two CTAs share the SM and one's epilogue overlaps
            // the other's MMAs; a grid that does not fill the machine gets the deeper pipeline instead.
            const long long ctas = (long long)((n_out + TC_BM - 1) / TC_BM) * ((T + 255) / 256) * splits;
            if (ctas > sm_count()) return tc_launch<256, 2>(mw, mx, p, splits, stream);
            return tc_launch<256, 4>(mw, mx, p, splits, stream);
        }
    }
}
