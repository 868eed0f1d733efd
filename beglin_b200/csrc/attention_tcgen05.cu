// Attention of prompt portions on the fifth-generation tensor cores (bfloat16, head size 64 or 128).
//
// One CTA takes a query block of up to 128 rows (consecutive tokens of one request x the query heads
// of one kv head) and walks all keys the block sees, a tile of 64 or of 128 keys at a time:
//   S = Q K^T      tcgen05.mma, Q and the key tile in shared memory (K-major, 128-byte swizzle), S in tensor
//                  memory: 256 columns hold the scores of four tiles of 64 keys or of two tiles of 128;
//   softmax        one thread per row: tcgen05.ld of the row's scores, scale, mask, running maximum and sum in
//                  float, P = exp2(S - m) as bfloat16, written by tcgen05.st over the columns the scores came
//                  from (two keys a column);
//   O += P V       tcgen05.mma with P as the left operand IN TENSOR MEMORY and the value tile as it lies in the
//                  cache (N-major) in shared memory; O in tensor memory.  When a row's maximum has grown by more
//                  than a factor of 256, its O is rescaled by tcgen05.ld / tcgen05.st before the product is issued.
// The softmax of a tile is a chain of latencies (the load from tensor memory, the maximum, the exponentials, the
// store of P) that one warp per SM sub-partition cannot hide.  So there are TWO groups of four softmax warps, each
// with a running maximum, a sum and an accumulator O in tensor memory of its own, as if the keys had been cut into
// two sets; the two are joined when all tiles are done
// (O = (O_0 2^(m_0 - m) + O_1 2^(m_1 - m)) / (l_0 2^(m_0 - m) + l_1 2^(m_1 - m))).  With tiles of 128 keys a tile
// is cut in two halves, one for each group; with tiles of 64 keys the groups take the tiles in turns.
// Tiles of 128 keys cost the tensor cores less per key (an MMA of 64 key columns takes as long as one of 128), tiles
// of 64 have four tiles under way instead of two and waste less on the tile at the diagonal: the narrow ones win up
// to about 24,000 keys.
// Keys and values come from the pages by TMA (cp.async.bulk.tensor over the page pool seen as a 2-D tensor
// [rows, head_dim], boxes of one page x 64 features, 128-byte swizzle), each through a ring of 256 keys of its own:
// a stage of the keys is free as soon as its scores are done, a stage of the values after the second product.
// Issuing an asynchronous operation (a copy, an MMA, a commit) costs the issuing thread a few hundred cycles, and a
// loader's turn for one tile is a chain of such operations that takes longer than the tensor cores need for the
// tile.  So the roles are spread over fourteen warps: warp 0 issues S = Q K^T, warp 6 issues O += P V, warps 5 and 12
// copy the keys of the even and the odd tiles, warps 7 and 13 the values, warps 1-4 and 8-11 are the two softmax
// groups.  A tile of values at the ragged end of the keys is completed by its loader (rows that the block must not
// see are zeroed, so that 0 * garbage cannot be NaN) before it is released.
// Every wait on an mbarrier is bounded in time and records BG_STATUS_TIMEOUT.
//
// The result is the finished row, out[t, h, :] = O / l, as in attention_mma.cu's rows arrangement.
#include "page_tma.cuh"

namespace bg {

constexpr int AT_BM = 128;                 // rows per CTA
// From this many keys on, tiles of 128 keys (BEGLIN_B200_ATTN_WIDE_FROM overrides the measured default).
inline int& at_wide_from() {
    static int v = [] { const char* e = getenv("BEGLIN_B200_ATTN_WIDE_FROM"); return (e && atoi(e) > 0) ? atoi(e) : 24576; }();
    return v;
}
// Stages of the key and value rings: 256 keys each.
constexpr int AT_THREADS = 448;            // warps 0 and 6: MMA issue; warps 1-4 and 8-11: softmax; warps 5, 7, 12, 13: loaders
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

__device__ __forceinline__ bool at_elect() {
    unsigned one;
    asm volatile("{\n .reg .pred p;\n elect.sync _|p, 0xffffffff;\n selp.u32 %0, 1, 0, p;\n}\n" : "=r"(one));
    return one != 0;
}
__device__ __forceinline__ float at_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

template <int HD, int AT_BK>
__global__ void __launch_bounds__(AT_THREADS)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_kv, AttnTcParams p) {
    constexpr int AT_HALF = AT_BK / 2, AT_STAGES = 256 / AT_BK;
    constexpr int NSB = AT_STAGES;                       // score buffers in tensor memory: tiles whose scores may be under way
    // How the two groups of softmax warps share the keys.  Tiles of 128 keys: every tile is cut in two halves, one for
    // each group.  Tiles of 64 keys: the groups take turns, the first the even tiles and the second the odd ones, so a
    // group's turn (the load of the scores, the store of P, the barriers: a few hundred cycles that do not depend on
    // the number of keys) comes once per 128 keys in both arrangements.
    constexpr bool ALT = AT_BK == 64;
    constexpr int GK = ALT ? AT_BK : AT_HALF;            // keys of a tile that one group takes
    constexpr int CB = HD / 64;                          // 64-feature column blocks of a row
    constexpr int Q_BYTES = CB * AT_BM * 128;
    constexpr int KV_BLOCK = AT_BK * 128;                // one column block of a key or value tile
    constexpr int KV_BYTES = CB * KV_BLOCK;
    // tensor memory: S in NSB buffers of AT_BK columns, 256 in all (the first half of a buffer's columns are the first
    // group's keys, the second half the second group's; a group's P, two bfloat16 a column, takes the first half of
    // its half), and an accumulator O of 128 columns for each group.  With tiles of 64 keys four tiles' scores are
    // under way at once, so that a group's softmax finds its next scores waiting: the chain product -> load ->
    // exponentials -> store -> product of one tile, with a barrier's latency at every arrow, is hidden behind three others.
    constexpr unsigned TMEM_COLS = 512;
    constexpr unsigned O_COL = 256;
    extern __shared__ unsigned char at_raw[];
    unsigned char* base = (unsigned char*)(((uintptr_t)at_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = base;
    unsigned char* k_s = q_s + Q_BYTES;
    unsigned char* v_s = k_s + AT_STAGES * KV_BYTES;
    // A commit costs its thread hundreds of cycles, so one commit serves every reader of an event: s_full[b] tells the
    // softmax warps that the scores of a tile are there AND the key loader that the tile's stage is free (a stage of
    // the rings and a score buffer have the same number); pv_done[b] tells the score issuer that buffer b may be
    // overwritten, the softmax warps that O may be rescaled, and the value loader that the stage is free.
    __shared__ __align__(8) unsigned long long k_full[AT_STAGES], v_full[AT_STAGES], kv_landed[AT_STAGES];
    __shared__ __align__(8) unsigned long long s_full[NSB], p_full[2 * NSB], pv_done[NSB], o_ready;    // p_full: [2 buffer + group]
    __shared__ float2 ml_other[AT_BM];                   // the second group's running maximum and sum of every row, for the join
    __shared__ unsigned tmem_sh;
    __shared__ int failed;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    // the blocks with the most keys (the last ones of a prompt) are handed out first, for every kv head, so that
    // the short ones fill the machine's last wave
    const int kvh = blockIdx.x, qb = (int)gridDim.y - 1 - (int)blockIdx.y;
    if (tid == 0) {
        for (int s = 0; s < AT_STAGES; ++s) {
            mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1); mbar_init(&kv_landed[s], 1);
        }
        for (int b = 0; b < NSB; ++b) { mbar_init(&s_full[b], 1); mbar_init(&pv_done[b], 1); }
        for (int b = 0; b < 2 * NSB; ++b) mbar_init(&p_full[b], 4);       // one arrival per softmax warp of a group
        mbar_init(&o_ready, 1);
        failed = 0;
        mbar_init_fence();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_sh)), "r"(TMEM_COLS) : "memory");
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
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = tmem_sh;
    // The kernel behind this one may be scheduled only now that this CTA holds its tensor memory: it takes all 512
    // columns, and a CTA of the successor that came to the same SM first and allocated a few would then wait for
    // this kernel to end while this CTA waits for its columns.
    pdl_launch();

    if (warp == 0 || warp == 6) {
        // ------------------------------------------------------------------ MMA issuers: warp 0 the scores, warp 6 the values
        // The whole warp runs the loop and one elected lane issues: addresses and descriptors then stay in
        // uniform registers, which keeps the issue of one small MMA to a few cycles.  P, the left operand of the
        // second product, lies in tensor memory, so that MMA reads only its value tile from shared memory (with
        // both operands there, a 128 x 128 x 16 MMA asks for all of an SM's shared-memory bandwidth).
        constexpr unsigned idesc_qk = instr_desc_bf16(AT_BM, AT_BK, 0);
        constexpr unsigned idesc_pv = instr_desc_bf16(AT_BM, HD, 1);
        const unsigned q_addr = smem_u32(q_s);
        bool ok = true;
        auto wait_all = [&](unsigned long long* bar, unsigned parity) {
            return __all_sync(0xffffffffu, mbar_wait(bar, parity)) != 0;
        };
        if (warp == 0) {
            // scores: S[b] = Q K(i)^T as soon as the keys have landed and both groups' P of the buffer's last tile
            // have been used up
            for (int i = 0; i < n_tiles && ok; ++i) {
                const int st = i % AT_STAGES, b = i % NSB;
                // (which of the two waits comes first is measured: with four score buffers the older event, the
                // buffer's release, first: 234 -> 227 us at 8,192 tokens; with two buffers the keys first: 812
                // against 864 us at 16,384 tokens)
                if (ALT) {
                    if (i >= NSB) ok = wait_all(&pv_done[b], ((i / NSB) - 1) & 1);
                    if (ok) ok = wait_all(&k_full[st], (i / AT_STAGES) & 1);
                } else {
                    ok = wait_all(&k_full[st], (i / AT_STAGES) & 1);
                    if (ok && i >= NSB) ok = wait_all(&pv_done[b], ((i / NSB) - 1) & 1);
                }
                if (!ok) break;
                tc_fence_after();
                const unsigned k_addr = smem_u32(k_s + st * KV_BYTES);
                if (at_elect()) {
#pragma unroll
                    for (int ks = 0; ks < HD / 16; ++ks) {
                        const unsigned off = (ks & 3) * 32;
                        tc_mma(tmem + (unsigned)b * AT_BK, smem_desc_sw128(q_addr + (ks >> 2) * (AT_BM * 128) + off),
                               smem_desc_sw128(k_addr + (ks >> 2) * KV_BLOCK + off), idesc_qk, ks > 0 ? 1u : 0u);
                    }
                    tc_commit(&s_full[b]);
                }
                __syncwarp();
            }
        } else {
            // values: O[g] += P(i, g) V(i, g) once group g's softmax warps have written their half of P
            for (int i = 0; i < n_tiles && ok; ++i) {
                const int st = i % AT_STAGES, b = i % NSB;
                ok = wait_all(&v_full[st], (i / AT_STAGES) & 1);
                const unsigned v_addr = smem_u32(v_s + st * KV_BYTES);
                if constexpr (ALT) {
                    const int g = i & 1;
                    if (ok) ok = wait_all(&p_full[b], (i / NSB) & 1);
                    if (!ok) break;
                    tc_fence_after();
                    if (at_elect()) {
#pragma unroll
                        for (int ks = 0; ks < AT_BK / 16; ++ks)
                            tc_mma_ts(tmem + O_COL + 128u * (unsigned)g, tmem + (unsigned)b * AT_BK + (unsigned)ks * 8,
                                      smem_desc_sw128_nmajor(v_addr + ks * 2048, KV_BLOCK, 1024), idesc_pv, (i >= 2 || ks > 0) ? 1u : 0u);
                        tc_commit(&pv_done[b]);
                    }
                    __syncwarp();
                } else {
                for (int g = 0; g < 2 && ok; ++g) {
                    ok = wait_all(&p_full[2 * b + g], (i / NSB) & 1);
                    if (!ok) break;
                    tc_fence_after();
                    if (at_elect()) {
#pragma unroll
                        for (int ks = 0; ks < AT_HALF / 16; ++ks)
                            tc_mma_ts(tmem + O_COL + 128u * (unsigned)g, tmem + (unsigned)b * AT_BK + (unsigned)g * AT_HALF + (unsigned)ks * 8,
                                      smem_desc_sw128_nmajor(v_addr + (g * (AT_HALF / 16) + ks) * 2048, KV_BLOCK, 1024), idesc_pv,
                                      (i > 0 || ks > 0) ? 1u : 0u);
                        if (g == 1) tc_commit(&pv_done[b]);
                    }
                    __syncwarp();
                }
                }
            }
            if (ok) { if (at_elect()) tc_commit(&o_ready); }
            __syncwarp();
        }
        if (!ok && lane == 0) atomicExch(&failed, 1);
    } else if (warp <= 4 || (warp >= 8 && warp <= 11)) {
        // ------------------------------------------------------------------ softmax: one thread per row, in each of two groups;
        // group 0 (warps 1-4) takes the first 64 keys of every tile, group 1 (warps 8-11) the last 64
        const int grp = warp >= 8 ? 1 : 0;
        const unsigned o_col = O_COL + 128u * (unsigned)grp;
        const int quarter = warp & 3;                    // the tensor-memory lanes this warp may touch
        const int r = quarter * 32 + lane;
        const unsigned lane_addr = (unsigned)(quarter * 32) << 16;
        const bool real = r < n_rows;
        const int pos = real ? pos_first + r / group : -1;
        const int lo = (real && p.window > 0) ? max(0, pos - p.window + 1) : 0;
        const int warp_pos_min = __reduce_min_sync(0xffffffffu, real ? pos : 0x7fffffff);
        const int warp_lo_max = __reduce_max_sync(0xffffffffu, lo);
        float m = -INFINITY, l = 0.0f;
        bool ok = true;
        const int i_first = ALT ? grp : 0;                   // this group's first tile
        for (int i = i_first; i < n_tiles && ok; i += (ALT ? 2 : 1)) {
            const int b = i % NSB;
            const unsigned s_col = (unsigned)b * AT_BK + (ALT ? 0u : (unsigned)grp * AT_HALF);    // this group's scores of the tile, and its P
            const int key0 = (tile0 + i) * AT_BK + (ALT ? 0 : grp * AT_HALF);
            ok = mbar_wait(&s_full[b], (i / NSB) & 1);
            if (!ok) break;
            tc_fence_after();
            float s[GK];
            if constexpr (GK == 64) tc_ld64(tmem + lane_addr + s_col, s);
            else tc_ld32(tmem + lane_addr + s_col, s);
            // only a half that some row of the warp sees in part is masked element by element
            float tm[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (key0 + GK - 1 > warp_pos_min || key0 < warp_lo_max) {
#pragma unroll
                for (int q = 0; q < GK; ++q) {
                    const int key = key0 + q;
                    s[q] = (key <= pos && key >= lo) ? s[q] : -INFINITY;
                    tm[q & 3] = fmaxf(tm[q & 3], s[q]);
                }
            } else {
#pragma unroll
                for (int q = 0; q < GK; ++q) tm[q & 3] = fmaxf(tm[q & 3], s[q]);
            }
            const float tmax = fmaxf(fmaxf(tm[0], tm[1]), fmaxf(tm[2], tm[3])) * p.scale_log2;   // the scale is positive
            // The reference maximum m moves only when some row of the warp outgrows it by more than 8 (a factor
            // of 256, harmless in float and bfloat16): then the rows' O and l are rescaled; otherwise the
            // exponentials keep the old reference and nothing that was accumulated needs touching.
            const bool grow = __any_sync(0xffffffffu, tmax > m + 8.0f) || (i == i_first);
            const float m_new = grow ? fmaxf(m, tmax) : m;
            const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
            const float corr = grow ? at_ex2(m - m_use) : 1.0f;
            float sums[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            float pk[GK / 2];                            // P: two keys a column
#pragma unroll
            for (int c = 0; c < GK / 2; ++c) {
                const float e0 = at_ex2(fmaf(s[2 * c], p.scale_log2, -m_use)), e1 = at_ex2(fmaf(s[2 * c + 1], p.scale_log2, -m_use));
                sums[c & 3] += e0 + e1;
                const __nv_bfloat162 h2 = __floats2bfloat162_rn(e0, e1);
                pk[c] = __uint_as_float(*reinterpret_cast<const unsigned*>(&h2));
            }
            const float sum = (sums[0] + sums[1]) + (sums[2] + sums[3]);
            l = l * corr + sum;
            m = m_new;
            // rows whose maximum grew: O *= corr, once this group's product before this one has landed
            const int prev = ALT ? i - 2 : i - 1;
            if (prev >= 0 && grow) {
                ok = mbar_wait(&pv_done[prev % NSB], (prev / NSB) & 1);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    float t[32];
                    tc_ld32(tmem + lane_addr + o_col + c0, t);
#pragma unroll
                    for (int q = 0; q < 32; ++q) t[q] *= corr;
                    tc_st32(tmem + lane_addr + o_col + c0, t);
                }
            }
            if constexpr (GK == 64) tc_st32(tmem + lane_addr + s_col, pk);       // over the first half of the scores it came from
            else tc_st16(tmem + lane_addr + s_col, pk);
            tc_wait_st();
            tc_fence_before();
            __syncwarp();                                // every lane's P has been stored: one arrival for the warp
            if (lane == 0) mbar_arrive(&p_full[ALT ? b : 2 * b + grp]);
        }
        if (ok && n_tiles > 0) ok = mbar_wait(&o_ready, 0);
        if (!ok) atomicExch(&failed, 1);
        // the join of the two groups: the second hands its maximum and sum over, the first group's thread of the
        // same row (the same lanes of tensor memory) reads both accumulators
        if (grp == 1) ml_other[r] = make_float2(m, l);
        asm volatile("bar.sync 1, 256;\n" ::: "memory");
        if (grp == 0 && ok && n_tiles > 0) {
            tc_fence_after();
            const float2 other = ml_other[r];
            const float m_all = fmaxf(m, other.x);
            const float m_ref = (m_all == -INFINITY) ? 0.0f : m_all;
            const float a0 = at_ex2(m - m_ref), a1 = at_ex2(other.x - m_ref);
            const float l_all = l * a0 + other.y * a1;
            const float inv = (real && l_all > 0.0f) ? 1.0f / l_all : 0.0f;
            const float w0 = a0 * inv, w1 = a1 * inv;
            const bool has1 = !ALT || n_tiles > 1;       // with one tile the second group's accumulator was never written
            const int qi = real ? r / group : 0, g = real ? r - qi * group : 0;
            __nv_bfloat16* o = p.out + (size_t)(row0 + qi) * p.out_stride + (size_t)(kvh * group + g) * HD;
#pragma unroll
            for (int c0 = 0; c0 < HD; c0 += 32) {
                float t[32], u[32];
                tc_ld32(tmem + lane_addr + O_COL + c0, t);        // all lanes take part; only real rows store
                tc_ld32(tmem + lane_addr + O_COL + 128u + c0, u);
                if (real) {
#pragma unroll
                    for (int q = 0; q < 32; q += 8) {
                        float v8[8];
#pragma unroll
                        for (int k = 0; k < 8; ++k) v8[k] = t[q + k] * w0 + (has1 ? u[q + k] * w1 : 0.0f);
                        store8(o + c0 + q, v8);
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ loaders: TMA, a tile of keys at a time;
        // warps 5 and 12 bring the keys, warps 7 and 13 the values, each pair through a ring of stages of its own.
        // A loader's turn for one tile (page numbers, the barrier's byte count, the copies: each an operation of a
        // few hundred cycles, one after the other) takes longer than the tensor cores need for the tile, so two
        // warps share a ring: one takes the even tiles, the other the odd ones.
        const int which = (warp == 7 || warp == 13);
        const int lsub = warp >= 12;
        unsigned char* ring = which ? v_s : k_s;
        unsigned long long* full = which ? v_full : k_full;
        unsigned long long* empty = which ? pv_done : s_full;      // AT_STAGES == NSB: stage st is buffer st
        const int ps = p.page_size, sh = p.page_shift;   // the page size is a power of two
        const int n_pg = AT_BK >> sh;                    // pages per tile (page_size divides 64)
        bool ok = true;
        unsigned landed_phase = 0;                       // bit s: parity of stage s's "landed" barrier
        constexpr int ROUNDS = AT_BK / 32;               // a lane holds the page of up to ROUNDS of a tile's pages (pages of one key)
        auto fetch_pages = [&](int i, int (&pg)[ROUNDS]) {
            const int key0 = (tile0 + i) * AT_BK;
#pragma unroll
            for (int h = 0; h < ROUNDS; ++h) {
                const int k = h * 32 + lane;
                const int pi = (key0 >> sh) + k;
                pg[h] = -1;
                if (i < n_tiles && k < n_pg && pi < p.max_pages && key0 + k * ps < k_end && key0 + (k + 1) * ps > k_begin)
                    pg[h] = p.block_table[(size_t)req * p.max_pages + pi];
            }
        };
        int pg_next[ROUNDS];
        fetch_pages(lsub, pg_next);
        for (int i = lsub; i < n_tiles && ok; i += 2) {
            const int st = i % AT_STAGES;
            if (i >= AT_STAGES) {
                ok = mbar_wait(&empty[st], ((i / AT_STAGES) - 1) & 1);
                if (!ok) break;
            }
            const int key0 = (tile0 + i) * AT_BK;
            unsigned char* dst = ring + st * KV_BYTES;
            // page numbers of the tile (fetched one tile ahead): lanes 0..n_pg-1 hold one each, in rounds of 32
            int pg[ROUNDS];
#pragma unroll
            for (int h = 0; h < ROUNDS; ++h) pg[h] = pg_next[h];
            fetch_pages(i + 2, pg_next);
            unsigned have[ROUNDS];
            int n_have = 0;
#pragma unroll
            for (int h = 0; h < ROUNDS; ++h) {
                if (pg[h] >= p.num_pages) { if (p.status) atomicOr(p.status, BG_STATUS_BAD_PAGE); pg[h] = -1; }
                have[h] = __ballot_sync(0xffffffffu, pg[h] >= 0);
                n_have += __popc(have[h]);
            }
            // Key rows that no query may see need no care (their scores are masked, whatever they are); value rows
            // do: 0 * garbage can be NaN.  So a ragged tile of values lands on a barrier of its own, the rows
            // outside the range or in pages that are not held are zeroed, and only then is the tile released.
            const bool direct = !which || (n_have == n_pg && key0 >= k_begin && key0 + AT_BK <= k_end);
            unsigned long long* bar = direct ? &full[st] : &kv_landed[st];
            if (lane == 0) {
                if (n_have > 0) mbar_expect_tx(bar, (unsigned)n_have * ps * HD * 2);
                else if (direct) mbar_arrive(bar);
            }
            __syncwarp();
#pragma unroll
            for (int h = 0; h < ROUNDS; ++h) {
                if (pg[h] >= 0) {
                    const int row = ((pg[h] * 2 + which) * p.nkv + kvh) * ps;
#pragma unroll
                    for (int cb = 0; cb < CB; ++cb)
                        tma_load_2d(dst + cb * KV_BLOCK + (h * 32 + lane) * ps * 128, &map_kv, cb * 64, row, bar);
                }
            }
            if (!direct) {
                if (n_have > 0) {
                    ok = mbar_wait(&kv_landed[st], (landed_phase >> st) & 1);
                    landed_phase ^= 1u << st;
                    if (!ok) break;
                }
                for (int idx = lane; idx < AT_BK * (HD / 8); idx += 32) {
                    const int jrow = idx / (HD / 8), c = idx - jrow * (HD / 8);
                    const int key = key0 + jrow, k = jrow >> sh;
                    unsigned mask = have[0];
#pragma unroll
                    for (int h = 1; h < ROUNDS; ++h) mask = (k >> 5) == h ? have[h] : mask;
                    const int held = (mask >> (k & 31)) & 1;
                    if (!held || key < k_begin || key >= k_end)
                        *reinterpret_cast<uint4*>(dst + (c >> 3) * KV_BLOCK + jrow * 128 + (((c & 7) ^ (jrow & 7)) << 4)) = make_uint4(0, 0, 0, 0);
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(&full[st]);
            }
        }
        if (!ok) atomicExch(&failed, 1);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
    if (tid == 0 && failed && p.status) atomicOr(p.status, BG_STATUS_TIMEOUT);
}

template <int HD, int BK>
static int at_launch(const CUtensorMap& map, const AttnTcParams& p, int n_qblk, cudaStream_t stream) {
    auto kern = attention_tcgen05_kernel<HD, BK>;
    // Q, and two rings (keys, values) of 256 keys each
    const size_t smem = (size_t)(HD / 64) * AT_BM * 128 + (size_t)2 * 256 * (HD / 64) * 128 + 1024;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    e = launch(kern, dim3(p.nkv, n_qblk), dim3(AT_THREADS), smem, stream, map, p);
    if (e != cudaSuccess) return (int)e;
    return BG_OK;
}

}  // namespace bg

using namespace bg;

// Sets the number of keys from which tiles of 128 keys are walked (0 or less: leaves it) and returns the old one.
extern "C" int bg_attention_tc_wide_from(int keys) {
    const int old = at_wide_from();
    if (keys > 0) at_wide_from() = keys;
    return old;
}

// Rows (tokens) per query block for these sizes, or BG_ERR_UNSUPPORTED.
extern "C" int bg_attention_tc_plan(int group, int hd, int page_size, int* bq_out) {
    if ((hd != 64 && hd != 128) || group < 1 || group > 128) return BG_ERR_UNSUPPORTED;
    if (page_size < 1 || page_size > 64 || 64 % page_size != 0) return BG_ERR_UNSUPPORTED;
    *bq_out = 128 / group;
    return BG_OK;
}

extern "C" int bg_attention_tc(const void* q, int q_stride, const void* kv_pool, int num_pages, int page_size,
                               const int* block_table, int max_pages, const int* positions, const int* qblk, int n_qblk,
                               void* out, int out_stride, int nh, int nkv, int hd, int window, float scale, int max_position,
                               unsigned* status, cudaStream_t stream) {
    if (n_qblk <= 0) return BG_OK;
    if (nh % nkv != 0 || (hd != 64 && hd != 128) || nh / nkv > 128 || !(scale > 0.0f)) return BG_ERR_UNSUPPORTED;
    if (page_size < 1 || page_size > 64 || 64 % page_size != 0) return BG_ERR_UNSUPPORTED;
    if ((q_stride % 8) || (out_stride % 8) || ((uintptr_t)q % 16) || ((uintptr_t)kv_pool % 16) || ((uintptr_t)out % 16)) return BG_ERR_ALIGN;
    if (n_qblk > 65535) return BG_ERR_SHAPE;                 // the query blocks are the grid's second dimension
    AttnTcParams p;
    p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride; p.kv_pool = (const __nv_bfloat16*)kv_pool;
    p.num_pages = num_pages; p.page_size = page_size; p.page_shift = -1;
    for (int sh = 0; sh < 30; ++sh) if ((1 << sh) == page_size) p.page_shift = sh;
    p.block_table = block_table; p.max_pages = max_pages; p.positions = positions; p.qblk = qblk;
    p.out = (__nv_bfloat16*)out; p.out_stride = out_stride; p.nh = nh; p.nkv = nkv; p.group = nh / nkv;
    p.window = window; p.scale_log2 = scale * AT_LOG2E; p.status = status;
    CUtensorMap map;
    int rc = pt_pool_map(&map, kv_pool, num_pages, nkv, page_size, hd);
    if (rc != BG_OK) return rc;
    // tiles of 128 keys where a block may walk many of them (max_position bounds the positions of the step's rows)
    const bool wide = (window > 0 ? (window < max_position + 1 ? window : max_position + 1) : max_position + 1) >= at_wide_from();
    if (hd == 128) return wide ? at_launch<128, 128>(map, p, n_qblk, stream) : at_launch<128, 64>(map, p, n_qblk, stream);
    return wide ? at_launch<64, 128>(map, p, n_qblk, stream) : at_launch<64, 64>(map, p, n_qblk, stream);
}
