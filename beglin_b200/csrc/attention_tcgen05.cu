// Attention of prompt portions on the fifth-generation tensor cores (bfloat16, head size 64 or 128).
//
// One CTA takes a query block of up to 128 rows (consecutive tokens of one request x the query heads
// of one kv head) and walks all keys the block sees, 64 at a time:
//   S = Q K^T      tcgen05.mma, Q and the key tile in shared memory (K-major, 128-byte swizzle),
//                  S in tensor memory (two buffers of 64 columns);
//   softmax        128 threads, one per row: tcgen05.ld of the row's 64 scores, scale, mask, running
//                  maximum and sum in float, P = exp2(S - m) as bfloat16 into shared memory;
//   O += P V       tcgen05.mma, P K-major, the value tile as it lies in the cache (N-major), O in
//                  tensor memory (head_dim columns); when a row's maximum grows, its O is rescaled
//                  by tcgen05.ld / tcgen05.st before the product is issued.
// Keys and values come from the pages through cp.async: three loader warps, one per stage, each
// signs its stage as soon as its own copies have landed; one thread issues the MMAs.  Every wait on an mbarrier is bounded in time and records BG_STATUS_TIMEOUT.
//
// The result is the finished row, out[t, h, :] = O / l, as in attention_mma.cu's rows arrangement.
#include <cuda.h>

#include "common.cuh"

namespace bg {

constexpr int AT_BM = 128;                 // rows per CTA
constexpr int AT_BK = 64;                  // keys per tile
constexpr int AT_STAGES = 3;
constexpr int AT_THREADS = 256;            // warp 0: MMA; warps 1-4: softmax; warps 5-7: loaders, one per stage
constexpr int AT_LOADERS = 32;             // threads that sign a stage's "full" barrier
constexpr unsigned long long AT_WAIT_NS = 1000000000ull;
constexpr float AT_LOG2E = 1.4426950408889634f;

struct AttnTcParams {
    const __nv_bfloat16* q;
    int q_stride;
    const __nv_bfloat16* kv_pool;
    int num_pages, page_size, page_shift;
    const int* block_table;
    int max_pages;
    const int* positions;
    const int* qblk;        // [n][3] = (request, first row, number of token rows)
    __nv_bfloat16* out;
    int out_stride;
    int nh, nkv, group, window;
    float scale_log2;
    unsigned* status;
};

__device__ __forceinline__ unsigned at_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void at_mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(at_smem(bar)), "r"(count));
}
__device__ __forceinline__ void at_mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(at_smem(bar)) : "memory");
}
__device__ __forceinline__ bool at_mbar_wait(unsigned long long* bar, unsigned parity) {
    unsigned addr = at_smem(bar);
    unsigned long long t0 = 0;
    for (unsigned it = 0;; ++it) {
        unsigned done;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if ((it & 255u) == 255u) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > AT_WAIT_NS) return false;
        }
    }
}
__device__ __forceinline__ void at_fence_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void at_tc_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void at_tc_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void at_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(at_smem(bar)) : "memory");
}
__device__ __forceinline__ void at_mma(unsigned tmem_d, unsigned long long a, unsigned long long b, unsigned idesc, unsigned acc) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void at_ld32(unsigned taddr, float (&v)[32]) {
    unsigned r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void at_st32(unsigned taddr, const float (&v)[32]) {
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
__device__ __forceinline__ float at_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// Operand descriptors, 128-byte swizzle.  K-major: rows of 128 bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ unsigned long long at_desc_kmajor(unsigned addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((addr & 0x3FFFFu) >> 4);
    d |= (unsigned long long)(1024u >> 4) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}
// N-major (the value tile, stored [key][feature]): a swizzle atom is 64 features x 8 keys; `lbo` is the
// distance between atoms along the features, `sbo` along the keys.
__device__ __forceinline__ unsigned long long at_desc_nmajor(unsigned addr, unsigned lbo, unsigned sbo) {
    unsigned long long d = 0;
    d |= (unsigned long long)((addr & 0x3FFFFu) >> 4);
    d |= (unsigned long long)((lbo >> 4) & 0x3FFFu) << 16;
    d |= (unsigned long long)((sbo >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}
__host__ __device__ constexpr unsigned at_idesc(int m, int n, int b_nmajor) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)b_nmajor << 16) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}

template <int HD>
__global__ void __launch_bounds__(AT_THREADS)
attention_tcgen05_kernel(AttnTcParams p) {
    constexpr int CB = HD / 64;                          // 64-feature column blocks of a row
    constexpr int Q_BYTES = CB * AT_BM * 128;
    constexpr int KV_BLOCK = AT_BK * 128;                // one column block of a key or value tile
    constexpr int KV_BYTES = CB * KV_BLOCK;
    constexpr int P_BYTES = AT_BM * 128;
    constexpr unsigned TMEM_COLS = 256;                  // S: 2 x 64, O: HD (<= 128)
    constexpr unsigned O_COL = 128;
    extern __shared__ unsigned char at_raw[];
    unsigned char* base = (unsigned char*)(((uintptr_t)at_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = base;
    unsigned char* k_s = q_s + Q_BYTES;
    unsigned char* v_s = k_s + AT_STAGES * KV_BYTES;
    unsigned char* p_s = v_s + AT_STAGES * KV_BYTES;     // two buffers
    __shared__ __align__(8) unsigned long long kv_full[AT_STAGES], kv_empty[AT_STAGES];
    __shared__ __align__(8) unsigned long long s_full[2], s_empty[2], p_full[2], p_empty[2], o_ready;
    __shared__ unsigned tmem_sh;
    __shared__ int failed;

    pdl_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int qb = blockIdx.x, kvh = blockIdx.y;
    if (tid == 0) {
        for (int s = 0; s < AT_STAGES; ++s) { at_mbar_init(&kv_full[s], AT_LOADERS); at_mbar_init(&kv_empty[s], 1); }
        for (int b = 0; b < 2; ++b) {
            at_mbar_init(&s_full[b], 1); at_mbar_init(&s_empty[b], 128);
            at_mbar_init(&p_full[b], 128); at_mbar_init(&p_empty[b], 1);
        }
        at_mbar_init(&o_ready, 1);
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(at_smem(&tmem_sh)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    pdl_wait();
    const int req = p.qblk[qb * 3 + 0], row0 = p.qblk[qb * 3 + 1], nq = p.qblk[qb * 3 + 2];
    const int group = p.group;
    const int n_rows = nq * group;                       // <= 128
    const int pos_first = p.positions[row0];
    const int pos_last = pos_first + nq - 1;
    const int k_begin = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
    const int k_end = pos_last + 1;
    const int tile0 = k_begin / AT_BK;
    const int n_tiles = (k_end + AT_BK - 1) / AT_BK - tile0;

    // ---- Q into shared memory: row r, column block cb, 16-byte piece c at r*128 + ((c ^ (r & 7)) * 16)
    for (int idx = tid; idx < AT_BM * (HD / 8); idx += AT_THREADS) {
        const int r = idx / (HD / 8), c = idx - r * (HD / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < n_rows) {
            const int qi = r / group, g = r - qi * group;
            v = *reinterpret_cast<const uint4*>(p.q + (size_t)(row0 + qi) * p.q_stride + (size_t)(kvh * group + g) * HD + c * 8);
        }
        const int cb = c >> 3, cc = c & 7;
        *reinterpret_cast<uint4*>(q_s + cb * (AT_BM * 128) + r * 128 + ((cc ^ (r & 7)) << 4)) = v;
    }
    at_fence_async();
    at_tc_before();
    __syncthreads();
    at_tc_after();
    const unsigned tmem = tmem_sh;

    if (warp == 0) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr unsigned idesc_qk = at_idesc(AT_BM, AT_BK, 0);
            constexpr unsigned idesc_pv = at_idesc(AT_BM, HD, 1);
            const unsigned q_addr = at_smem(q_s);
            bool ok = true;
            auto issue_qk = [&](int i) {
                const int st = i % AT_STAGES, b = i & 1;
                ok = ok && at_mbar_wait(&kv_full[st], (i / AT_STAGES) & 1);
                if (ok && i >= 2) ok = at_mbar_wait(&s_empty[b], ((i >> 1) - 1) & 1);
                if (!ok) return;
                at_tc_after();
                const unsigned k_addr = at_smem(k_s + st * KV_BYTES);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {
                    const unsigned off = (ks >> 2) * 0 + (ks & 3) * 32;
                    at_mma(tmem + (unsigned)b * 64, at_desc_kmajor(q_addr + (ks >> 2) * (AT_BM * 128) + off),
                           at_desc_kmajor(k_addr + (ks >> 2) * KV_BLOCK + off), idesc_qk, ks > 0 ? 1u : 0u);
                }
                at_commit(&s_full[b]);
            };
            if (n_tiles > 0) issue_qk(0);
            for (int i = 0; i < n_tiles && ok; ++i) {
                if (i + 1 < n_tiles) issue_qk(i + 1);
                if (!ok) break;
                const int st = i % AT_STAGES, b = i & 1;
                ok = at_mbar_wait(&p_full[b], (i >> 1) & 1);
                if (!ok) break;
                at_tc_after();
                const unsigned p_addr = at_smem(p_s + b * P_BYTES);
                const unsigned v_addr = at_smem(v_s + st * KV_BYTES);
#pragma unroll
                for (int ks = 0; ks < AT_BK / 16; ++ks)
                    at_mma(tmem + O_COL, at_desc_kmajor(p_addr + ks * 32), at_desc_nmajor(v_addr + ks * 2048, KV_BLOCK, 1024),
                           idesc_pv, (i > 0 || ks > 0) ? 1u : 0u);
                at_commit(&kv_empty[st]);
                at_commit(&p_empty[b]);
            }
            if (ok) at_commit(&o_ready);
            else atomicExch(&failed, 1);
        }
    } else if (warp <= 4) {
        // ------------------------------------------------------------------ softmax: one thread per row
        const int quarter = warp & 3;                    // the tensor-memory lanes this warp may touch
        const int r = quarter * 32 + lane;
        const unsigned lane_addr = (unsigned)(quarter * 32) << 16;
        const bool real = r < n_rows;
        const int pos = real ? pos_first + r / group : -1;
        const int lo = (real && p.window > 0) ? max(0, pos - p.window + 1) : 0;
        float m = -INFINITY, l = 0.0f;
        bool ok = true;
        for (int i = 0; i < n_tiles && ok; ++i) {
            const int b = i & 1;
            const int key0 = (tile0 + i) * AT_BK;
            ok = at_mbar_wait(&s_full[b], (i >> 1) & 1);
            if (!ok) break;
            at_tc_after();
            float s[64];
            {
                float t[32];
                at_ld32(tmem + lane_addr + (unsigned)b * 64, t);
#pragma unroll
                for (int j = 0; j < 32; ++j) s[j] = t[j];
                at_ld32(tmem + lane_addr + (unsigned)b * 64 + 32, t);
#pragma unroll
                for (int j = 0; j < 32; ++j) s[32 + j] = t[j];
            }
            at_tc_before();
            at_mbar_arrive(&s_empty[b]);                 // the scores are in registers
            float tmax = -INFINITY;
#pragma unroll
            for (int j = 0; j < 64; ++j) {
                const int key = key0 + j;
                const bool seen = key <= pos && key >= lo;
                s[j] = seen ? s[j] * p.scale_log2 : -INFINITY;
                tmax = fmaxf(tmax, s[j]);
            }
            const float m_new = fmaxf(m, tmax);
            const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
            const float corr = at_ex2(m - m_use);
            float sum = 0.0f;
            if (i >= 2) { ok = at_mbar_wait(&p_empty[b], ((i >> 1) - 1) & 1); if (!ok) break; }
            unsigned char* prow = p_s + b * P_BYTES + r * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                float e[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) { e[j] = at_ex2(s[c * 8 + j] - m_use); sum += e[j]; }
                uint4 pk;
                __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                for (int j = 0; j < 4; ++j) h2[j] = __floats2bfloat162_rn(e[2 * j], e[2 * j + 1]);
                *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) = pk;
            }
            l = l * corr + sum;
            m = m_new;
            // rows whose maximum grew: O *= corr, once the previous product has landed
            if (i > 0 && __any_sync(0xffffffffu, corr < 1.0f)) {
                ok = at_mbar_wait(&p_empty[(i - 1) & 1], ((i - 1) >> 1) & 1);
                if (!ok) break;
                at_tc_after();
#pragma unroll
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    float t[32];
                    at_ld32(tmem + lane_addr + O_COL + c0, t);
#pragma unroll
                    for (int j = 0; j < 32; ++j) t[j] *= corr;
                    at_st32(tmem + lane_addr + O_COL + c0, t);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
                at_tc_before();
            }
            at_fence_async();                            // P (written through the generic proxy) for the MMA
            at_mbar_arrive(&p_full[b]);
        }
        if (ok && n_tiles > 0) ok = at_mbar_wait(&o_ready, 0);
        if (!ok) atomicExch(&failed, 1);
        if (ok && real && n_tiles > 0) {
            at_tc_after();
        }
        if (ok && n_tiles > 0) {
            at_tc_after();
            const float inv = real ? 1.0f / l : 0.0f;
            const int qi = real ? r / group : 0, g = real ? r - qi * group : 0;
            __nv_bfloat16* o = p.out + (size_t)(row0 + qi) * p.out_stride + (size_t)(kvh * group + g) * HD;
#pragma unroll
            for (int c0 = 0; c0 < HD; c0 += 32) {
                float t[32];
                at_ld32(tmem + lane_addr + O_COL + c0, t);        // all lanes take part; only real rows store
                if (real) {
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        float v8[8];
#pragma unroll
                        for (int k = 0; k < 8; ++k) v8[k] = t[j + k] * inv;
                        store8(o + c0 + j, v8);
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ loaders: warp 5 + s owns stage s
        const int st = warp - 5;
        const size_t page_elems = (size_t)2 * p.nkv * p.page_size * HD;
        const size_t v_off = (size_t)p.nkv * p.page_size * HD;
        constexpr int PIECES = HD / 8;                   // 16-byte pieces per key row
        unsigned char* kd = k_s + st * KV_BYTES;
        unsigned char* vd = v_s + st * KV_BYTES;
        const int c = lane % PIECES, cb = c >> 3, cc = c & 7;
        bool ok = true;
        for (int i = st; i < n_tiles; i += AT_STAGES) {
            if (i >= AT_STAGES) {
                ok = at_mbar_wait(&kv_empty[st], ((i / AT_STAGES) - 1) & 1);
                if (!ok) break;
            }
            const int key0 = (tile0 + i) * AT_BK;
            // lane copies piece lane % PIECES of keys lane / PIECES, + 32 / PIECES, ...: whole rows per warp access
            for (int j = lane / PIECES; j < AT_BK; j += 32 / PIECES) {
                const int key = key0 + j;
                const unsigned off = cb * KV_BLOCK + j * 128 + ((cc ^ (j & 7)) << 4);
                const __nv_bfloat16* src = nullptr;
                if (key >= k_begin && key < k_end) {
                    const int pi = p.page_shift >= 0 ? key >> p.page_shift : key / p.page_size;
                    const int slot = p.page_shift >= 0 ? key & (p.page_size - 1) : key - pi * p.page_size;
                    const int page = p.block_table[(size_t)req * p.max_pages + pi];
                    if (page < 0 || page >= p.num_pages) {
                        if (p.status) atomicOr(p.status, BG_STATUS_BAD_PAGE);
                    } else {
                        src = p.kv_pool + (size_t)page * page_elems + ((size_t)kvh * p.page_size + slot) * HD + c * 8;
                    }
                }
                if (src) {
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(at_smem(kd + off)), "l"(src) : "memory");
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(at_smem(vd + off)), "l"(src + v_off) : "memory");
                } else {
                    *reinterpret_cast<uint4*>(kd + off) = make_uint4(0, 0, 0, 0);
                    *reinterpret_cast<uint4*>(vd + off) = make_uint4(0, 0, 0, 0);
                }
            }
            asm volatile("cp.async.commit_group;\n" ::: "memory");
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
            at_fence_async();                            // the tile is read through the async proxy
            at_mbar_arrive(&kv_full[st]);
        }
        if (!ok) atomicExch(&failed, 1);
    }
    at_tc_before();
    __syncthreads();
    if (warp == 0) {
        at_tc_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
    if (tid == 0 && failed && p.status) atomicOr(p.status, BG_STATUS_TIMEOUT);
}

template <int HD>
static int at_launch(const AttnTcParams& p, int n_qblk, cudaStream_t stream) {
    auto kern = attention_tcgen05_kernel<HD>;
    const size_t smem = (size_t)(HD / 64) * AT_BM * 128 + (size_t)2 * AT_STAGES * (HD / 64) * AT_BK * 128 + 2 * AT_BM * 128 + 1024;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    e = launch(kern, dim3(n_qblk, p.nkv), dim3(AT_THREADS), smem, stream, p);
    if (e != cudaSuccess) return (int)e;
    return BG_OK;
}

}  // namespace bg

using namespace bg;

// Rows (tokens) per query block for these sizes, or BG_ERR_UNSUPPORTED.
extern "C" int bg_attention_tc_plan(int group, int hd, int* bq_out) {
    if ((hd != 64 && hd != 128) || group < 1 || group > 128) return BG_ERR_UNSUPPORTED;
    *bq_out = 128 / group;
    return BG_OK;
}

extern "C" int bg_attention_tc(const void* q, int q_stride, const void* kv_pool, int num_pages, int page_size,
                               const int* block_table, int max_pages, const int* positions, const int* qblk, int n_qblk,
                               void* out, int out_stride, int nh, int nkv, int hd, int window, float scale,
                               unsigned* status, cudaStream_t stream) {
    if (n_qblk <= 0) return BG_OK;
    if (nh % nkv != 0 || (hd != 64 && hd != 128) || nh / nkv > 128) return BG_ERR_UNSUPPORTED;
    if ((q_stride % 8) || (out_stride % 8) || ((uintptr_t)q % 16) || ((uintptr_t)kv_pool % 16) || ((uintptr_t)out % 16)) return BG_ERR_ALIGN;
    if (nkv > 65535) return BG_ERR_SHAPE;
    AttnTcParams p;
    p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride; p.kv_pool = (const __nv_bfloat16*)kv_pool;
    p.num_pages = num_pages; p.page_size = page_size; p.page_shift = -1;
    for (int sh = 0; sh < 30; ++sh) if ((1 << sh) == page_size) p.page_shift = sh;
    p.block_table = block_table; p.max_pages = max_pages; p.positions = positions; p.qblk = qblk;
    p.out = (__nv_bfloat16*)out; p.out_stride = out_stride; p.nh = nh; p.nkv = nkv; p.group = nh / nkv;
    p.window = window; p.scale_log2 = scale * AT_LOG2E; p.status = status;
    return hd == 128 ? at_launch<128>(p, n_qblk, stream) : at_launch<64>(p, n_qblk, stream);
}
