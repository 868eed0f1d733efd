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
#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

namespace bg {

constexpr int TC_BM = 128;                 // output features per CTA (MMA M)
constexpr int TC_BK = 64;                  // k per stage: 64 bf16 = 128 bytes = one swizzle row
constexpr int TC_THREADS = 192;            // warp 0: TMA, warp 1: MMA + tensor memory, warps 2-5: epilogue
constexpr unsigned long long TC_WAIT_NS = 1000000000ull;   // a wait gives up after one second

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity.  Returns false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
    unsigned addr = smem_u32(bar);
    unsigned long long t0 = 0;
    for (unsigned it = 0;; ++it) {
        unsigned done;
        // the hint lets the hardware park the thread (up to 2 us) instead of polling: polls of many waiting
        // threads would crowd the shared-memory pipeline that the copies of other warps need
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(done) : "r"(addr), "r"(parity), "r"(2000u) : "memory");
        if (done) return true;
        if ((it & 15u) == 15u) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > TC_WAIT_NS) return false;
        }
    }
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc, unsigned idesc,
                                       unsigned accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld16(unsigned taddr, unsigned (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

// Shared-memory operand descriptor: K-major tile whose rows are 128 bytes, 128-byte swizzle; groups
// of 8 rows are 1024 bytes apart.
__device__ __forceinline__ unsigned long long smem_desc_sw128(unsigned smem_addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_addr & 0x3FFFFu) >> 4);          // start address
    d |= (unsigned long long)(1024u >> 4) << 32;                     // stride between 8-row groups
    d |= 1ull << 46;                                                 // descriptor version of sm_100
    d |= 2ull << 61;                                                 // 128-byte swizzle
    return d;
}

// kind::f16 instruction descriptor: float accumulator, bfloat16 A and B, both K-major, M x N.
__host__ __device__ constexpr unsigned instr_desc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}

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

// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

// A [rows, K] bfloat16 matrix with row stride ld (elements), cut into boxes of box_rows x 64.
static int make_map(CUtensorMap* map, const void* base, long long rows, int K, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return BG_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? BG_OK : BG_ERR_SHAPE;
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
    static std::mutex mu;
    static std::map<std::tuple<const void*, int, int, int>, CUtensorMap> w_maps;
    CUtensorMap mw, mx;
    {
        std::lock_guard<std::mutex> g(mu);
        auto key = std::make_tuple(W, n_out, K, ldw);
        auto it = w_maps.find(key);
        if (it == w_maps.end()) {
            int rc = make_map(&mw, W, n_out, K, ldw, TC_BM);
            if (rc != BG_OK) return rc;
            w_maps.emplace(key, mw);
        } else {
            mw = it->second;
        }
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
            if (ctas > 148) return tc_launch<256, 2>(mw, mx, p, splits, stream);
            return tc_launch<256, 4>(mw, mx, p, splits, stream);
        }
    }
}
