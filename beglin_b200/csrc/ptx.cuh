// The one set of inline-PTX wrappers that the kernels of this library share: mbarriers with bounded waits, TMA
// copies, the tcgen05 instructions (fences, commit, MMA with either left operand, loads and stores of tensor
// memory), operand and instruction descriptors, and the driver entry point that encodes tensor maps.
#pragma once
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace bg {

constexpr unsigned long long MBAR_WAIT_NS = 1000000000ull;   // a wait on a barrier gives up after one second

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

// ------------------------------------------------------------------------------------------------ mbarriers
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
// One arrival that also adds to the bytes the current phase waits for.
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Adds to the bytes that the current phase waits for, without arriving.
__device__ __forceinline__ void mbar_expect_only(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity.  Returns false when the limit (MBAR_WAIT_NS) ran out, or as
// soon as *gave_up (a flag in shared memory that the first thread to give up sets) is non-zero.
// The time hint lets the hardware park the thread (up to that many ns) instead of polling: the polls of a hundred
// waiting threads would crowd the shared-memory pipeline that the copies of other warps go through.
template <unsigned HINT_NS = 2000>
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, volatile int* gave_up = nullptr) {
    const unsigned addr = smem_u32(bar);
    unsigned long long t0 = 0;
    for (unsigned it = 0;; ++it) {
        unsigned done;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(done) : "r"(addr), "r"(parity), "r"(HINT_NS) : "memory");
        if (done) return true;
        if ((it & 15u) == 15u) {
            if (gave_up && *gave_up) return false;
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > MBAR_WAIT_NS) { if (gave_up) *gave_up = 1; return false; }
        }
    }
}

// ------------------------------------------------------------------------------------------------ TMA
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
// A 5-D box at (0, 0, 0, 0, u): everything one (page, kv head) holds, see pt_page_map.
__device__ __forceinline__ void tma_load_5d_last(void* smem_dst, const CUtensorMap* map, int u, unsigned long long* bar) {
    asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %2, %2, %2, %3}], [%4];\n"
                 ::"r"(smem_u32(smem_dst)), "l"(map), "r"(0), "r"(u), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];\n"
                 ::"l"(map), "r"(smem_u32(smem_src)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];\n"
                 ::"l"(map), "r"(smem_u32(smem_src)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(map) : "memory");
}
// Writes of this thread to shared memory become visible to the asynchronous proxy (TMA, tcgen05.mma).
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// ------------------------------------------------------------------------------------------------ tcgen05
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
// D (tensor memory) (+)= A (shared memory) B (shared memory)
__device__ __forceinline__ void tc_mma(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc, unsigned idesc,
                                       unsigned accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// The same with the left operand in tensor memory (row i in lane i, two bfloat16 of consecutive k a column).
__device__ __forceinline__ void tc_mma_ts(unsigned tmem_d, unsigned tmem_a, unsigned long long bdesc, unsigned idesc,
                                          unsigned accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
// Loads of 16 or 32 consecutive columns of the warp's 32 lanes; the _nowait forms leave the wait to the caller,
// so that several loads are on their way before the one wait.
__device__ __forceinline__ void tc_ld16(unsigned taddr, unsigned (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    tc_wait_ld();
}
#define BG_TC_LD32_ASM(base, r, off)                                                                                        \
    asm volatile(                                                                                                           \
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"                   \
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"                                        \
        : "=r"(r[off + 0]), "=r"(r[off + 1]), "=r"(r[off + 2]), "=r"(r[off + 3]), "=r"(r[off + 4]), "=r"(r[off + 5]),       \
          "=r"(r[off + 6]), "=r"(r[off + 7]), "=r"(r[off + 8]), "=r"(r[off + 9]), "=r"(r[off + 10]), "=r"(r[off + 11]),     \
          "=r"(r[off + 12]), "=r"(r[off + 13]), "=r"(r[off + 14]), "=r"(r[off + 15]), "=r"(r[off + 16]), "=r"(r[off + 17]), \
          "=r"(r[off + 18]), "=r"(r[off + 19]), "=r"(r[off + 20]), "=r"(r[off + 21]), "=r"(r[off + 22]), "=r"(r[off + 23]), \
          "=r"(r[off + 24]), "=r"(r[off + 25]), "=r"(r[off + 26]), "=r"(r[off + 27]), "=r"(r[off + 28]), "=r"(r[off + 29]), \
          "=r"(r[off + 30]), "=r"(r[off + 31])                                                                              \
        : "r"(base))
__device__ __forceinline__ void tc_ld32_nowait(unsigned taddr, unsigned (&r)[32]) { BG_TC_LD32_ASM(taddr, r, 0); }
__device__ __forceinline__ void tc_ld32(unsigned taddr, float (&v)[32]) {
    unsigned r[32];
    BG_TC_LD32_ASM(taddr, r, 0);
    tc_wait_ld();
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tc_ld64(unsigned taddr, float (&v)[64]) {
    unsigned r[64];
    BG_TC_LD32_ASM(taddr, r, 0);
    BG_TC_LD32_ASM(taddr + 32, r, 32);
    tc_wait_ld();
#pragma unroll
    for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tc_st32(unsigned taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
          "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
          "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
          "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
          "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
          "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
          "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
}
__device__ __forceinline__ void tc_st16(unsigned taddr, const float (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
          "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
          "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15]))
        : "memory");
}

// Shared-memory operand descriptors, 128-byte swizzle.  K-major: rows of 128 bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ unsigned long long smem_desc_sw128(unsigned smem_addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_addr & 0x3FFFFu) >> 4);          // start address
    d |= (unsigned long long)(1024u >> 4) << 32;                     // stride between 8-row groups
    d |= 1ull << 46;                                                 // descriptor version of sm_100
    d |= 2ull << 61;                                                 // 128-byte swizzle
    return d;
}
// N-major (a tile stored [k][n], such as values [key][feature]): a swizzle atom is 64 n x 8 k; `lbo` is the
// distance between atoms along n, `sbo` along k.
__device__ __forceinline__ unsigned long long smem_desc_sw128_nmajor(unsigned smem_addr, unsigned lbo, unsigned sbo) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_addr & 0x3FFFFu) >> 4);
    d |= (unsigned long long)((lbo >> 4) & 0x3FFFu) << 16;
    d |= (unsigned long long)((sbo >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}
// kind::f16 instruction descriptor: float accumulator, bfloat16 A and B, A K-major, B K-major or N-major, M x N.
__host__ __device__ constexpr unsigned instr_desc_bf16(int m, int n, int b_nmajor = 0) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)b_nmajor << 16) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}

// ------------------------------------------------------------------------------------------------ tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point (the library links no driver stub), or null.
inline EncodeTiledFn encode_fn() {
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

}  // namespace bg
