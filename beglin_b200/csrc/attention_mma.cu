// Tensor-core attention over the paged cache for bfloat16 queries and caches (head sizes 64, 128).
//
// Same contract as attention.cu: a CTA takes (query block, kv head, split of keys) and writes, for
// every (row, head) that sees a key of the split, an unnormalised output with its running maximum
// and sum; attention_merge joins the splits.  Scores, softmax and the output accumulators are float;
// the two products of a 16-key block run as mma.sync m16n8k16 on bfloat16 operands with float
// accumulation.  Keys and values are brought from the pages into shared memory three stages of 64
// keys deep.  When the page size divides 64 a fifth warp does nothing but ask for them by TMA (one box
// per page, kv head and 64 features: one instruction moves kilobytes, where a warp's 16-byte copies
// in flight are too few to keep up with HBM, and the address arithmetic of a stage, a long chain for
// one thread, stays off the four computing warps' path); stages are handed over through mbarriers.
// Else the four warps copy with 16-byte cp.async themselves.  The layout is the one the TMA's 128-byte
// swizzle gives: per 64 features a block of rows of 128 bytes, the 16-byte column XORed with the
// key's low bits, so that ldmatrix reads without bank conflicts.
//
// Two arrangements of the four warps:
//   rows:  the query block has up to 64 rows (tokens x heads of the group); warp w owns rows
//          16w..16w+15 and walks all keys of a stage (prompt portions).
//   keys:  the query block is ONE token (<= 16 heads in the group); warp w owns every fourth stage of
//          64 keys (stage s lands in buffer s % 4, which is warp s % 4's), walks it alone, and the four
//          partial results are joined in shared memory at the end (decoding: a stage is a long chain of
//          dependent steps for one warp, so four of them run side by side, each with 64 keys' worth of
//          independent MMAs, and no barrier of the CTA stands between two stages).  With at most 8 heads
//          per kv head the products are turned around (SWAP): the 16 keys of a block are the M side of
//          the instruction and the heads the N side of 8, S^T = K Q^T and O^T = V^T P^T, which halves
//          the MMAs of a stage (the heads fill 6 of 8 columns instead of 6 of 16 rows); P^T reaches its
//          operand layout through movmatrix.
#include "page_tma.cuh"

namespace bg {

constexpr int AM_THREADS = 128;             // the computing warps
constexpr int AM_ALL = AM_THREADS + 32;     // and the warp that asks for the copies
constexpr int AM_STAGE_KEYS = 64;
// Stages of 64 keys in flight per CTA: 3 for prompt portions, 4 (a buffer per warp) for decoding.
constexpr int AM_TABLE = 128;              // block-table entries held in shared memory at a time
constexpr float AM_LOG2E = 1.4426950408889634f;
constexpr float AM_LN2 = 0.6931471805599453f;

struct AttnMmaParams {
    const __nv_bfloat16* q;
    int q_stride;
    const __nv_bfloat16* kv_pool;
    int num_pages, page_size;
    int page_shift;         // log2(page_size) when it is a power of two, else -1
    const int* block_table;
    int max_pages;
    const int* positions;
    const int* qblk;
    float* part_o;
    float* part_ml;
    int max_splits;
    int nh, nkv, group;
    int window, split;
    float scale_log2;       // scale * log2(e)
    unsigned* status;
    __nv_bfloat16* out;     // rows arrangement only: when set, a CTA walks ALL keys of its block and writes
    int out_stride;         // the finished rows here (no partial results, no merge)
    int use_tma;            // pages are copied as TMA boxes (the page size divides 64)
    int whole_pages;        // a page is a stage (64 positions): keys and values of a stage come in ONE box
};

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
    unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
    unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x by the hardware's approximation (relative error about 2^-22; -inf gives 0).
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
// transposes an 8x8 matrix of 16-bit values held one 32-bit register (two values) per lane
__device__ __forceinline__ unsigned movmatrix_trans(unsigned a) {
    unsigned d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// Byte offset of (row, 16-byte column c) in a tile whose rows are HD bf16 wide.
template <int HD> __device__ __forceinline__ int swz(int row, int c) { return row * (HD * 2) + ((c ^ (row & 7)) << 4); }
// key and value tiles: a block of 64 rows x 128 bytes per 64 features
__device__ __forceinline__ int swz_kv(int row, int c) {
    return (c >> 3) * (AM_STAGE_KEYS * 128) + row * 128 + (((c & 7) ^ (row & 7)) << 4);
}

template <int HD, bool BY_KEYS, int AM_STAGES, bool SWAP>
__global__ void __launch_bounds__(AM_ALL)
attention_mma_kernel(const __grid_constant__ CUtensorMap map_kv, const __grid_constant__ CUtensorMap map_page, AttnMmaParams p) {
    constexpr int CH = HD / 8;                 // 16-byte columns per row
    constexpr int KSTEPS = HD / 16;            // k-steps of q.k
    constexpr int NT_O = HD / 8;               // 8-wide column tiles of the output
    constexpr int STAGE_BYTES = AM_STAGE_KEYS * HD * 2;
    constexpr int Q_ROWS = BY_KEYS ? 16 : 64;
    extern __shared__ unsigned char sm_raw[];
    unsigned char* sm = (unsigned char*)(((uintptr_t)sm_raw + 1023) & ~(uintptr_t)1023);   // the swizzle wants 1024
    unsigned char* k_s = sm;                                   // stage b: keys at b * 2 * STAGE_BYTES, [HD / 64][64][128 bytes],
    unsigned char* v_s = k_s + STAGE_BYTES;                    // and its values right behind them, the same
    unsigned char* q_s = k_s + 2 * AM_STAGES * STAGE_BYTES;    // [Q_ROWS][HD]
    constexpr int BUF_BYTES = 2 * STAGE_BYTES;
    __shared__ __align__(8) unsigned long long full_bar[AM_STAGES], empty_bar[AM_STAGES];
    __shared__ int gave_up;

    pdl_launch();
    // Decoding (keys arrangement): the kernel before this one wrote the step's queries and the ONE new key
    // and value of every request; positions, block tables and all older keys and values are from earlier
    // steps.  So everything up to the first copies of old pages happens before the wait for that kernel, and
    // when it has finished the data is already on its way (or here).
    if (!BY_KEYS) pdl_wait();
    const int qb = blockIdx.x, kvh = blockIdx.y, sp = blockIdx.z;
    // without a list of query blocks, block i is row i of request i (a step of single tokens)
    const int req = p.qblk ? p.qblk[qb * 3 + 0] : qb, row0 = p.qblk ? p.qblk[qb * 3 + 1] : qb;
    const int nq = p.qblk ? p.qblk[qb * 3 + 2] : 1;
    if (nq <= 0) return;
    const int group = p.group;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_rows = nq * group;             // <= 64 (rows) or <= 16 (keys)

    // ---- everything that does not depend on the positions goes out first, so that the positions, the
    // queries and the block table arrive in one round trip: the queries of the block into shared memory
    // (rows beyond n_rows are zero) ...
    const int pos_first = p.positions[row0];
    const int pos_last = p.positions[row0 + nq - 1];
    auto load_queries = [&](int first, int step) {
        for (int idx = first; idx < Q_ROWS * CH; idx += step) {
            int r = idx / CH, c = idx - r * CH;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < n_rows) {
                int qi = BY_KEYS ? 0 : r / group, g = r - qi * group;
                v = *reinterpret_cast<const uint4*>(p.q + (size_t)(row0 + qi) * p.q_stride + (size_t)(kvh * group + g) * HD + c * 8);
            }
            *reinterpret_cast<uint4*>(q_s + swz<HD>(r, c)) = v;
        }
    };
    if (!BY_KEYS) load_queries(tid, AM_ALL);
    // ... and the block-table entries of 128 pages at a time, kept in shared memory so that a stage's
    // copies start without a table load of their own (a stage of 64 keys never straddles two such groups).
    // The group fetched here is the one the first keys of this CTA's range lie in when there is no window.
    __shared__ int table_s[AM_TABLE];
    if (tid == 0) {
        for (int s = 0; s < AM_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], BY_KEYS ? 1 : AM_THREADS / 32); }
        gave_up = 0;
        mbar_init_fence();
    }
    const bool direct = !BY_KEYS && p.out != nullptr;
    const int split = keys_per_split(p.split, pos_last + 1, (int)gridDim.z);
    const int pre_key = direct ? 0 : sp * split;
    const int pre_group = (p.page_shift >= 0 ? pre_key >> p.page_shift : pre_key / p.page_size) / AM_TABLE;
    for (int i = tid; i < AM_TABLE; i += AM_ALL) {
        const int pi = pre_group * AM_TABLE + i;
        table_s[i] = pi < p.max_pages ? p.block_table[(size_t)req * p.max_pages + pi] : -1;
    }

    const int lo_first = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
    const int k_begin = direct ? lo_first : max(sp * split, lo_first);
    const int k_end = direct ? pos_last + 1 : min((sp + 1) * split, pos_last + 1);
    if (k_begin >= k_end) return;

    // ---- stage loader: thread t copies 16-byte pieces of key rows of K and of V
    const int first_stage_key = (k_begin / AM_STAGE_KEYS) * AM_STAGE_KEYS;
    const int n_stage = (k_end - first_stage_key + AM_STAGE_KEYS - 1) / AM_STAGE_KEYS;
    const int last_page = (k_end - 1) / p.page_size;
    int table_group = (first_stage_key / p.page_size) / AM_TABLE;
    if (table_group != pre_group) table_group = -1;               // a window moved the range: fetched by the loader
    __syncthreads();                           // table_s and the barriers are ready (and q_s, rows arrangement)
    auto compute_sync = [] { asm volatile("bar.sync 1, %0;\n" ::"n"(AM_THREADS) : "memory"); };   // the four computing warps
    if (BY_KEYS && warp < AM_THREADS / 32) {
        pdl_wait();                            // the queries come from the kernel before this one
        load_queries(tid, AM_THREADS);
        compute_sync();
    }
    if (warp == AM_THREADS / 32) {
        // ---- the copying warp.  A page of a stage is 2 * HD / 64 boxes (keys and values, 64 features each);
        // box o of the stage is lane o's, so that one instruction of the warp asks for up to 32 boxes (what
        // costs is the instruction, not the box).  Pages that lie wholly outside the range of keys are left
        // out; rows outside it are zeroed by the computing warps once the stage has landed.
        if (!p.use_tma) return;
        constexpr int PER_PAGE = 2 * (HD / 64);
        const int ps = p.page_size, shift = p.page_shift;
        const int n_box = (AM_STAGE_KEYS >> shift) * PER_PAGE;
        const int* table = p.block_table + (size_t)req * p.max_pages;
        auto page_of = [&](int s, int o) {               // the page that box o of stage s comes from, or -1
            const int key_lo = first_stage_key + s * AM_STAGE_KEYS + (o / PER_PAGE) * ps;
            if (s >= n_stage || o >= n_box || key_lo >= k_end || key_lo + ps <= k_begin || (key_lo >> shift) >= p.max_pages) return -1;
            return table[key_lo >> shift];
        };
        // stages of old keys only may be asked for before the kernel ahead has finished: all but the one that
        // holds the newest position
        const int n_early = BY_KEYS ? min(AM_STAGES, k_end == pos_last + 1 ? n_stage - 1 : n_stage) : 0;
        int next_page = page_of(0, p.whole_pages ? lane * PER_PAGE : lane);
        for (int s = 0; s < n_stage; ++s) {
            if (BY_KEYS && s == n_early) pdl_wait();
            const int buf = s % AM_STAGES;
            int page = next_page;
            next_page = page_of(s + 1, p.whole_pages ? lane * PER_PAGE : lane);   // fetched while this stage's copies go out
            if (s >= AM_STAGES && !mbar_wait<4000>(&empty_bar[buf], ((s / AM_STAGES) - 1) & 1, &gave_up)) {
                if (p.status) atomicOr(p.status, BG_STATUS_TIMEOUT);
                return;
            }
            unsigned char* kd = k_s + buf * BUF_BYTES;
            if (p.whole_pages) {                         // lane 0 holds the stage's page
                if (lane == 0) {
                    if (page >= p.num_pages) { if (p.status) atomicOr(p.status, BG_STATUS_BAD_PAGE); page = -1; }
                    if (page >= 0) {
                        mbar_expect_tx(&full_bar[buf], BUF_BYTES);
                        tma_load_5d_last(kd, &map_page, page * 2 * p.nkv + kvh, &full_bar[buf]);
                    } else {
                        mbar_arrive(&full_bar[buf]);
                    }
                }
                continue;
            }
            for (int h = 0; h * 32 < n_box; ++h) {       // more than one round only for pages of fewer than 8 positions
                const int o = h * 32 + lane;
                if (h > 0) page = page_of(s, o);
                if (page >= p.num_pages) { if (p.status) atomicOr(p.status, BG_STATUS_BAD_PAGE); page = -1; }
                const unsigned have = __ballot_sync(0xffffffffu, page >= 0);
                if (lane == 0 && have) mbar_expect_only(&full_bar[buf], (unsigned)__popc(have) * ps * 128);
                __syncwarp();
                if (page >= 0) {
                    const int k = o / PER_PAGE, rem = o % PER_PAGE, which = rem / (HD / 64), cb = rem % (HD / 64);
                    tma_load_2d(kd + which * STAGE_BYTES + cb * (AM_STAGE_KEYS * 128) + k * ps * 128, &map_kv, cb * 64,
                              ((page * 2 + which) * p.nkv + kvh) * ps, &full_bar[buf]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&full_bar[buf]);   // the one arrival the phase waits for, after every expect_tx
        }
        return;
    }
    const size_t page_elems = (size_t)2 * p.nkv * p.page_size * HD;
    const size_t v_off = (size_t)p.nkv * p.page_size * HD;
    auto load_stage = [&](int s) {
        if (p.use_tma) return;                                   // the copying warp's job
        if (s < n_stage) {
            const int stage_key0 = first_stage_key + s * AM_STAGE_KEYS;
            const int group_of_stage = (stage_key0 / p.page_size) / AM_TABLE;
            if (group_of_stage != table_group) {                 // uniform over the computing warps
                compute_sync();
                table_group = group_of_stage;
                const int base = table_group * AM_TABLE;
                for (int i = tid; i < AM_TABLE; i += AM_THREADS)
                    table_s[i] = (base + i <= last_page) ? p.block_table[(size_t)req * p.max_pages + base + i] : -1;
                compute_sync();
            }
            const int buf = s % AM_STAGES;
            unsigned char* kd = k_s + buf * BUF_BYTES;
            unsigned char* vd = v_s + buf * BUF_BYTES;
            // thread t copies 16-byte piece t % CH of rows t / CH, t / CH + ROWS_PER_PASS, ...: the lanes of
            // a warp read whole rows, so every 32-byte sector is asked for once
            constexpr int ROWS_PER_PASS = AM_THREADS / CH;
            const int c = tid % CH;
#pragma unroll
            for (int j = tid / CH; j < AM_STAGE_KEYS; j += ROWS_PER_PASS) {
                const int key = stage_key0 + j;
                const __nv_bfloat16* src = nullptr;
                if (key >= k_begin && key < k_end) {
                    const int pi = p.page_shift >= 0 ? key >> p.page_shift : key / p.page_size;
                    const int slot = p.page_shift >= 0 ? key & (p.page_size - 1) : key - pi * p.page_size;
                    const int page = table_s[pi - table_group * AM_TABLE];
                    if (page < 0 || page >= p.num_pages) {
                        if (p.status) atomicOr(p.status, BG_STATUS_BAD_PAGE);
                    } else {
                        src = p.kv_pool + (size_t)page * page_elems + ((size_t)kvh * p.page_size + slot) * HD + c * 8;
                    }
                }
                if (src) {
                    cp_async16(kd + swz_kv(j, c), src);
                    cp_async16(vd + swz_kv(j, c), src + v_off);
                } else {                                         // a key outside the range: zeros
                    *reinterpret_cast<uint4*>(kd + swz_kv(j, c)) = make_uint4(0, 0, 0, 0);
                    *reinterpret_cast<uint4*>(vd + swz_kv(j, c)) = make_uint4(0, 0, 0, 0);
                }
            }
        }
        cp_async_commit();
    };
    if (!BY_KEYS) {
#pragma unroll
        for (int s = 0; s < AM_STAGES - 1; ++s) load_stage(s);
    }

    // ---- this warp's query fragments and row bookkeeping
    const int row_base = BY_KEYS ? 0 : warp * 16;
    unsigned qf[KSTEPS][4];
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
        int r = row_base + (lane & 15);
        int c = ks * 2 + (lane >> 4);
        ldmatrix_x4(qf[ks], q_s + swz<HD>(r, c));
    }
    int pos_r[2], lo_r[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        int r = row_base + (lane >> 2) + h * 8;
        if (r < n_rows) {
            pos_r[h] = pos_first + r / group;
            lo_r[h] = p.window > 0 ? max(0, pos_r[h] - p.window + 1) : 0;
        } else {
            pos_r[h] = -1; lo_r[h] = 0;
        }
    }
    // the span of keys that the rows of this warp can see at all, and the span that ALL its rows see
    const int warp_row_hi = min(n_rows - 1, row_base + 15);
    const int warp_pos_hi = row_base < n_rows ? pos_first + warp_row_hi / group : -1;
    const int warp_pos_lo = pos_first + min(row_base, n_rows - 1) / group;
    const int warp_lo = p.window > 0 ? max(0, warp_pos_lo - p.window + 1) : 0;
    const int warp_lo_hi = p.window > 0 ? max(0, warp_pos_hi - p.window + 1) : 0;
    // byte offsets inside a 16-key block that do not change from block to block: the XOR of the swizzle
    // depends on the row's low three bits, which for a given lane are the same in every block
    int koff[KSTEPS], voff[NT_O / 2];
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks)
        koff[ks] = swz_kv((lane & 7) + ((lane >> 4) << 3), ks * 2 + ((lane >> 3) & 1));
#pragma unroll
    for (int t2 = 0; t2 < NT_O / 2; ++t2)
        voff[t2] = swz_kv((lane & 7) + (((lane >> 3) & 1) << 3), t2 * 2 + (lane >> 4));

    float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.0f, 0.0f};
    float o[NT_O][4];
#pragma unroll
    for (int t = 0; t < NT_O; ++t) { o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.0f; }
    // SWAP: the heads are the N side.  This lane's heads are r0 = 2 (lane % 4) and r0 + 1; qsw holds Q as the B
    // operand, ot the transposed output: ot[db][e] is feature db * 16 + lane / 4 + 8 (e >> 1) of head r0 + (e & 1).
    unsigned qsw[KSTEPS][2];
    float ot[HD / 16][4];
    int koff_a[KSTEPS], voff_a[HD / 16];
    if (SWAP) {
#pragma unroll
        for (int ks2 = 0; ks2 < KSTEPS / 2; ++ks2) {
            unsigned r4[4];
            ldmatrix_x4(r4, q_s + swz<HD>(lane & 7, ks2 * 4 + (lane >> 3)));
            qsw[2 * ks2][0] = r4[0]; qsw[2 * ks2][1] = r4[1]; qsw[2 * ks2 + 1][0] = r4[2]; qsw[2 * ks2 + 1][1] = r4[3];
        }
#pragma unroll
        for (int db = 0; db < HD / 16; ++db) { ot[db][0] = ot[db][1] = ot[db][2] = ot[db][3] = 0.0f; }
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) koff_a[ks] = swz_kv((lane & 7) + (((lane >> 3) & 1) << 3), ks * 2 + (lane >> 4));
#pragma unroll
        for (int db = 0; db < HD / 16; ++db) voff_a[db] = swz_kv((lane & 7) + ((lane >> 4) << 3), db * 2 + ((lane >> 3) & 1));
    }

    constexpr int KB = 4;                               // 16-key blocks of a stage
    constexpr int BLOCK_BYTES = 16 * 128;               // 16 keys further down, in every block of 64 features
    for (int s = BY_KEYS ? warp : 0; s < n_stage; s += (BY_KEYS ? AM_THREADS / 32 : 1)) {
        if (!BY_KEYS) load_stage(s + AM_STAGES - 1);
        const int buf = s % AM_STAGES;
        unsigned char* kt = k_s + buf * BUF_BYTES;
        unsigned char* vt = v_s + buf * BUF_BYTES;
        const int stage_key0 = first_stage_key + s * AM_STAGE_KEYS;
        // who reads this stage: the warp alone (keys arrangement) or the four warps together
        const int t0 = BY_KEYS ? lane : tid, nt = BY_KEYS ? 32 : AM_THREADS;
        if (p.use_tma) {
            // A wait that runs out records it and goes on (with whatever the buffer holds; the host raises on
            // the status): every thread then still reaches the barriers below.
            if (!mbar_wait<4000>(&full_bar[buf], (s / AM_STAGES) & 1, &gave_up) && p.status) atomicOr(p.status, BG_STATUS_TIMEOUT);
            if (stage_key0 < k_begin || stage_key0 + AM_STAGE_KEYS > k_end) {      // uniform over the readers
                // whole pages were copied: rows outside the range of keys become zeros (a value row that no
                // query sees must not hold garbage, since 0 * NaN is NaN)
                for (int idx = t0; idx < AM_STAGE_KEYS * CH; idx += nt) {
                    const int j = idx / CH, c = idx - j * CH;
                    if (stage_key0 + j < k_begin || stage_key0 + j >= k_end) {
                        *reinterpret_cast<uint4*>(kt + swz_kv(j, c)) = make_uint4(0, 0, 0, 0);
                        *reinterpret_cast<uint4*>(vt + swz_kv(j, c)) = make_uint4(0, 0, 0, 0);
                    }
                }
                fence_proxy_async();
                if (BY_KEYS) __syncwarp(); else compute_sync();
            }
        } else if (BY_KEYS) {
            // pages of a size that does not divide 64: the warp copies its stage itself, 16 bytes at a time
            for (int idx = lane; idx < AM_STAGE_KEYS * CH; idx += 32) {
                const int j = idx / CH, c = idx - j * CH, key = stage_key0 + j;
                const __nv_bfloat16* src = nullptr;
                if (key >= k_begin && key < k_end) {
                    const int pi = key / p.page_size, slot = key - pi * p.page_size;
                    const int page = pi < p.max_pages ? p.block_table[(size_t)req * p.max_pages + pi] : -1;
                    if (page < 0 || page >= p.num_pages) {
                        if (p.status) atomicOr(p.status, BG_STATUS_BAD_PAGE);
                    } else {
                        src = p.kv_pool + (size_t)page * page_elems + ((size_t)kvh * p.page_size + slot) * HD + c * 8;
                    }
                }
                if (src) {
                    cp_async16(kt + swz_kv(j, c), src);
                    cp_async16(vt + swz_kv(j, c), src + v_off);
                } else {
                    *reinterpret_cast<uint4*>(kt + swz_kv(j, c)) = make_uint4(0, 0, 0, 0);
                    *reinterpret_cast<uint4*>(vt + swz_kv(j, c)) = make_uint4(0, 0, 0, 0);
                }
            }
            cp_async_commit();
            cp_async_wait<0>();
            __syncwarp();
        } else {
            cp_async_wait<AM_STAGES - 1>();
            compute_sync();
        }
        // this warp's keys of the stage: [w_key0, w_key0 + 16 * KB)
        const int w_key0 = stage_key0;
        const int vis_lo = max(max(w_key0, k_begin), warp_lo);                   // keys some row of the warp sees
        const int vis_hi = min(min(w_key0 + 16 * KB, k_end), warp_pos_hi + 1);
        if (SWAP && vis_lo < vis_hi) {
            // ---- S^T = K Q^T: per block of 16 keys a 16 x 8 tile; c[kb][e]: key kb * 16 + lane / 4 + 8 (e >> 1), head r0 + (e & 1)
            float c[KB][4];
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) { c[kb][0] = c[kb][1] = c[kb][2] = c[kb][3] = 0.0f; }
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
                for (int kb = 0; kb < KB; ++kb) {
                    unsigned a[4];
                    ldmatrix_x4(a, kt + kb * BLOCK_BYTES + koff_a[ks]);
                    mma_bf16(c[kb], a, qsw[ks][0], qsw[ks][1]);
                }
            }
            const int r0 = 2 * (lane & 3);
            const int pos = pos_first, lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
            const bool all_seen = w_key0 >= k_begin && w_key0 + 16 * KB <= k_end && w_key0 >= lo && w_key0 + 16 * KB - 1 <= pos;
            float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int kb = 0; kb < KB; ++kb)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = w_key0 + kb * 16 + (lane >> 2) + 8 * (e >> 1);
                    const bool ok = all_seen || (key <= pos && key >= lo && key >= k_begin && key < k_end);
                    const float v = (ok && r0 + (e & 1) < n_rows) ? c[kb][e] * p.scale_log2 : -INFINITY;
                    c[kb][e] = v;
                    tmax[e & 1] = fmaxf(tmax[e & 1], v);
                }
            float corr[2], m_use[2], psum[2] = {0.0f, 0.0f};
#pragma unroll
            for (int j = 0; j < 2; ++j) {                                        // the keys of a head lie across lane / 4
                tmax[j] = fmaxf(tmax[j], __shfl_xor_sync(0xffffffffu, tmax[j], 4));
                tmax[j] = fmaxf(tmax[j], __shfl_xor_sync(0xffffffffu, tmax[j], 8));
                tmax[j] = fmaxf(tmax[j], __shfl_xor_sync(0xffffffffu, tmax[j], 16));
                const float m_new = fmaxf(m_r[j], tmax[j]);
                m_use[j] = (m_new == -INFINITY) ? 0.0f : m_new;
                corr[j] = ex2(m_r[j] - m_use[j]);
                m_r[j] = m_new;
            }
#pragma unroll
            for (int kb = 0; kb < KB; ++kb)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    c[kb][e] = ex2(c[kb][e] - m_use[e & 1]);
                    psum[e & 1] += c[kb][e];
                }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                psum[j] += __shfl_xor_sync(0xffffffffu, psum[j], 4);
                psum[j] += __shfl_xor_sync(0xffffffffu, psum[j], 8);
                psum[j] += __shfl_xor_sync(0xffffffffu, psum[j], 16);
                l_r[j] = l_r[j] * corr[j] + psum[j];
            }
#pragma unroll
            for (int db = 0; db < HD / 16; ++db) {
                ot[db][0] *= corr[0]; ot[db][1] *= corr[1]; ot[db][2] *= corr[0]; ot[db][3] *= corr[1];
            }
            // ---- O^T += V^T P^T: P^T of a block as the B operand (keys x heads) through a transpose of the packed tile
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
                const unsigned b0 = movmatrix_trans(pack_bf16(c[kb][0], c[kb][1]));
                const unsigned b1 = movmatrix_trans(pack_bf16(c[kb][2], c[kb][3]));
#pragma unroll
                for (int db = 0; db < HD / 16; ++db) {
                    unsigned a[4];
                    ldmatrix_x4_trans(a, vt + kb * BLOCK_BYTES + voff_a[db]);
                    mma_bf16(ot[db], a, b0, b1);
                }
            }
        }
        if (!SWAP && vis_lo < vis_hi) {                                          // warp-uniform
            // ---- scores of 16 rows x 16*KB keys
            // (k-step outermost, so the 2*KB accumulators form independent chains of dependent MMAs)
            float sc[2 * KB][4];
#pragma unroll
            for (int j = 0; j < 2 * KB; ++j) { sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.0f; }
            const unsigned char* kwarp = kt;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
                for (int kbi = 0; kbi < KB; ++kbi) {
                    unsigned kf[4];
                    ldmatrix_x4(kf, kwarp + kbi * BLOCK_BYTES + koff[ks]);
                    mma_bf16(sc[2 * kbi], qf[ks], kf[0], kf[1]);
                    mma_bf16(sc[2 * kbi + 1], qf[ks], kf[2], kf[3]);
                }
            }
            // ---- scale; mask only where a row of the warp does not see a key of the warp's span
            const bool all_seen = w_key0 >= k_begin && w_key0 + 16 * KB <= k_end && w_key0 >= warp_lo_hi &&
                                  w_key0 + 16 * KB - 1 <= warp_pos_lo && row_base + 15 < n_rows;
            float tmax[2] = {-INFINITY, -INFINITY};
            if (all_seen) {
#pragma unroll
                for (int j = 0; j < 2 * KB; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        sc[j][e] *= p.scale_log2;
                        tmax[e >> 1] = fmaxf(tmax[e >> 1], sc[j][e]);
                    }
            } else {
#pragma unroll
                for (int j = 0; j < 2 * KB; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = w_key0 + j * 8 + (lane & 3) * 2 + (e & 1);
                        const int h = e >> 1;
                        const bool ok = key <= pos_r[h] && key >= lo_r[h] && key >= k_begin && key < k_end;
                        const float v = ok ? sc[j][e] * p.scale_log2 : -INFINITY;
                        sc[j][e] = v;
                        tmax[h] = fmaxf(tmax[h], v);
                    }
            }
            float corr[2], m_use[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 1));
                tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 2));
                const float m_new = fmaxf(m_r[h], tmax[h]);
                m_use[h] = (m_new == -INFINITY) ? 0.0f : m_new;                  // a row that has seen nothing yet
                corr[h] = ex2(m_r[h] - m_use[h]);                               // ex2(-inf) = 0
                m_r[h] = m_new;
            }
            float psum[2] = {0.0f, 0.0f};
#pragma unroll
            for (int j = 0; j < 2 * KB; ++j) {
                sc[j][0] = ex2(sc[j][0] - m_use[0]);
                sc[j][1] = ex2(sc[j][1] - m_use[0]);
                sc[j][2] = ex2(sc[j][2] - m_use[1]);
                sc[j][3] = ex2(sc[j][3] - m_use[1]);
                psum[0] += sc[j][0] + sc[j][1];
                psum[1] += sc[j][2] + sc[j][3];
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 1);
                psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 2);
                l_r[h] = l_r[h] * corr[h] + psum[h];
            }
#pragma unroll
            for (int t = 0; t < NT_O; ++t) {
                o[t][0] *= corr[0]; o[t][1] *= corr[0]; o[t][2] *= corr[1]; o[t][3] *= corr[1];
            }
            // ---- o += p . v, block by block (16 keys, all HD columns, two 8-wide column tiles per ldmatrix)
#pragma unroll
            for (int kbi = 0; kbi < KB; ++kbi) {
                unsigned pf[4];
                pf[0] = pack_bf16(sc[2 * kbi][0], sc[2 * kbi][1]);
                pf[1] = pack_bf16(sc[2 * kbi][2], sc[2 * kbi][3]);
                pf[2] = pack_bf16(sc[2 * kbi + 1][0], sc[2 * kbi + 1][1]);
                pf[3] = pack_bf16(sc[2 * kbi + 1][2], sc[2 * kbi + 1][3]);
                const unsigned char* vblock = vt + kbi * BLOCK_BYTES;
#pragma unroll
                for (int t2 = 0; t2 < NT_O / 2; ++t2) {
                    unsigned vf[4];
                    ldmatrix_x4_trans(vf, vblock + voff[t2]);
                    mma_bf16(o[t2 * 2 + 0], pf, vf[0], vf[1]);
                    mma_bf16(o[t2 * 2 + 1], pf, vf[2], vf[3]);
                }
            }
        }
        // the stage's buffer may be refilled
        if (p.use_tma) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[buf]);
        } else if (!BY_KEYS) {
            compute_sync();
        }
    }
    if (!p.use_tma && !BY_KEYS) cp_async_wait<0>();

    // ---- write the partial results
    if (direct) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            int r = row_base + (lane >> 2) + h * 8;
            if (r >= n_rows) continue;
            int qi = r / group, g = r - qi * group;
            const float inv = 1.0f / l_r[h];
            __nv_bfloat16* po = p.out + (size_t)(row0 + qi) * p.out_stride + (size_t)(kvh * group + g) * HD;
#pragma unroll
            for (int t = 0; t < NT_O; ++t)
                *reinterpret_cast<unsigned*>(po + t * 8 + (lane & 3) * 2) = pack_bf16(o[t][h * 2 + 0] * inv, o[t][h * 2 + 1] * inv);
        }
    } else if (!BY_KEYS) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            int r = row_base + (lane >> 2) + h * 8;
            if (r >= n_rows) continue;
            if (pos_r[h] < sp * split || lo_r[h] >= (sp + 1) * split) continue;
            int qi = r / group, g = r - qi * group;
            size_t prow = ((size_t)(row0 + qi) * p.nh + (size_t)kvh * group + g) * p.max_splits + sp;
            float* po = p.part_o + prow * HD;
#pragma unroll
            for (int t = 0; t < NT_O; ++t) {
                float2 v = make_float2(o[t][h * 2 + 0], o[t][h * 2 + 1]);
                *reinterpret_cast<float2*>(po + t * 8 + (lane & 3) * 2) = v;
            }
            if ((lane & 3) == 0) { p.part_ml[prow * 2 + 0] = m_r[h] * AM_LN2; p.part_ml[prow * 2 + 1] = l_r[h]; }
        }
    } else {
        // join the four warps' results: o_w, m_w, l_w -> shared memory (over the stage buffers, once every
        // warp has read its last keys and values from them)
        compute_sync();
        constexpr int HP = HD + 4;                                 // rows four floats apart from a multiple of 128 bytes:
        float* o_sh = reinterpret_cast<float*>(k_s);               // [4][16][HP]  the stores below meet no bank twice
        float* ml_sh = o_sh + 4 * 16 * HP;                         // [4][16][2]
        if (SWAP) {
            const int r0 = 2 * (lane & 3);
#pragma unroll
            for (int db = 0; db < HD / 16; ++db)
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    o_sh[((size_t)warp * 16 + r0 + (e & 1)) * HP + db * 16 + (lane >> 2) + 8 * (e >> 1)] = ot[db][e];
            if (lane < 4) {
#pragma unroll
                for (int j = 0; j < 2; ++j) { ml_sh[(warp * 16 + r0 + j) * 2 + 0] = m_r[j]; ml_sh[(warp * 16 + r0 + j) * 2 + 1] = l_r[j]; }
            }
        }
#pragma unroll
        for (int h = 0; h < 2 && !SWAP; ++h) {
            int r = (lane >> 2) + h * 8;
            float* dst = o_sh + ((size_t)warp * 16 + r) * HP;
#pragma unroll
            for (int t = 0; t < NT_O; ++t) {
                dst[t * 8 + (lane & 3) * 2 + 0] = o[t][h * 2 + 0];
                dst[t * 8 + (lane & 3) * 2 + 1] = o[t][h * 2 + 1];
            }
            if ((lane & 3) == 0) { ml_sh[(warp * 16 + r) * 2 + 0] = m_r[h]; ml_sh[(warp * 16 + r) * 2 + 1] = l_r[h]; }
        }
        compute_sync();
        const int pos = pos_first;
        const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
        if (!(pos < sp * split || lo >= (sp + 1) * split)) {
            // every thread takes one feature of all rows and works out the weights of the four warps' parts itself
            // (four exponentials a row: cheaper than a third barrier and a round through shared memory)
            if (tid < HD) {
                const int d = tid;
#pragma unroll 2
                for (int r = 0; r < n_rows; ++r) {
                    float mw[4], m = -INFINITY;
#pragma unroll
                    for (int w = 0; w < 4; ++w) { mw[w] = ml_sh[(w * 16 + r) * 2]; m = fmaxf(m, mw[w]); }
                    float acc = 0.0f, l = 0.0f;
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        const float f = (mw[w] == -INFINITY) ? 0.0f : exp2f(mw[w] - m);
                        acc = fmaf(o_sh[((size_t)w * 16 + r) * HP + d], f, acc);
                        l = fmaf(ml_sh[(w * 16 + r) * 2 + 1], f, l);
                    }
                    if (p.out) {                               // the only range of its request: the finished row
                        p.out[(size_t)row0 * p.out_stride + (size_t)(kvh * group + r) * HD + d] = __float2bfloat16_rn(acc / l);
                    } else {
                        const size_t prow = ((size_t)row0 * p.nh + (size_t)kvh * group + r) * p.max_splits + sp;
                        p.part_o[prow * HD + d] = acc;
                        if (d == 0) { p.part_ml[prow * 2 + 0] = m * AM_LN2; p.part_ml[prow * 2 + 1] = l; }
                    }
                }
            }
        }
    }
}

template <int HD, bool BY_KEYS, int STAGES>
static size_t am_smem_bytes() {
    return (size_t)(BY_KEYS ? 16 : 64) * HD * 2 + (size_t)2 * STAGES * AM_STAGE_KEYS * HD * 2 + 1024;
}

template <int HD, bool BY_KEYS, int STAGES, bool SWAP = false>
static int am_launch_stages(const CUtensorMap& map, const CUtensorMap& map5, const AttnMmaParams& p, int n_qblk, int n_splits, cudaStream_t stream) {
    auto kern = attention_mma_kernel<HD, BY_KEYS, STAGES, SWAP>;
    size_t smem = am_smem_bytes<HD, BY_KEYS, STAGES>();
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid(n_qblk, p.nkv, n_splits);
    e = launch(kern, grid, dim3(AM_ALL), smem, stream, map, map5, p);
    if (e != cudaSuccess) return (int)e;
    return BG_OK;
}

template <int HD, bool BY_KEYS>
static int am_launch(const CUtensorMap& map, const CUtensorMap& map5, const AttnMmaParams& p, int n_qblk, int n_splits, cudaStream_t stream) {
    if (BY_KEYS && p.group <= 8) return am_launch_stages<HD, BY_KEYS, AM_THREADS / 32, BY_KEYS>(map, map5, p, n_qblk, n_splits, stream);
    if (BY_KEYS) return am_launch_stages<HD, BY_KEYS, AM_THREADS / 32>(map, map5, p, n_qblk, n_splits, stream);   // a buffer per warp
    return am_launch_stages<HD, BY_KEYS, 3>(map, map5, p, n_qblk, n_splits, stream);
}

}  // namespace bg

using namespace bg;

// Whether the tensor-core kernel takes these sizes, and how many rows (tokens) a query block may
// hold: by_keys != 0 asks for the decoding arrangement (one token per block).
extern "C" int bg_attention_mma_plan(int group, int hd, int by_keys, int* bq_out) {
    if (hd != 64 && hd != 128) return BG_ERR_UNSUPPORTED;
    if (by_keys) {
        if (group > 16) return BG_ERR_UNSUPPORTED;
        *bq_out = 1;
    } else {
        if (group > 64) return BG_ERR_UNSUPPORTED;
        *bq_out = 64 / group;
    }
    return BG_OK;
}

extern "C" int bg_attention_mma_partial(const void* q, int q_stride, const void* kv_pool, int num_pages, int page_size,
                                        const int* block_table, int max_pages, const int* positions, const int* qblk,
                                        int n_qblk, float* part_o, float* part_ml, int max_splits, int n_splits_launch,
                                        int nh, int nkv, int hd, int window, int split, int by_keys, float scale,
                                        void* direct_out, int out_stride, unsigned* status, cudaStream_t stream) {
    if (n_qblk <= 0 || n_splits_launch <= 0) return BG_OK;
    if (direct_out && (n_splits_launch != 1 || (out_stride % 2) != 0)) return BG_ERR_SHAPE;
    if (nh % nkv != 0 || split % AM_STAGE_KEYS != 0 || (split <= 0 && !by_keys)) return BG_ERR_SHAPE;
    if (n_splits_launch > max_splits || n_splits_launch > 65535 || nkv > 65535) return BG_ERR_SHAPE;
    if ((q_stride % 8) != 0 || ((uintptr_t)q % 16) != 0 || ((uintptr_t)kv_pool % 16) != 0) return BG_ERR_ALIGN;
    AttnMmaParams p;
    p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride; p.kv_pool = (const __nv_bfloat16*)kv_pool;
    p.num_pages = num_pages; p.page_size = page_size; p.block_table = block_table;
    p.page_shift = -1;
    for (int sh = 0; sh < 30; ++sh) if ((1 << sh) == page_size) p.page_shift = sh; p.max_pages = max_pages;
    p.positions = positions; p.qblk = qblk; p.part_o = part_o; p.part_ml = part_ml; p.max_splits = max_splits;
    p.nh = nh; p.nkv = nkv; p.group = nh / nkv; p.window = window; p.split = split;
    p.scale_log2 = scale * AM_LOG2E; p.status = status;
    p.out = (__nv_bfloat16*)direct_out; p.out_stride = out_stride;
    if (by_keys ? p.group > 16 : p.group > 64) return BG_ERR_UNSUPPORTED;
    if (hd != 64 && hd != 128) return BG_ERR_UNSUPPORTED;
    CUtensorMap map;
    memset(&map, 0, sizeof(map));
    CUtensorMap map5;
    memset(&map5, 0, sizeof(map5));
    p.use_tma = pt_page_size_ok(page_size) && p.page_shift >= 0 && pt_pool_map(&map, kv_pool, num_pages, nkv, page_size, hd) == BG_OK;
    p.whole_pages = p.use_tma && page_size == AM_STAGE_KEYS && pt_page_map(&map5, kv_pool, num_pages, nkv, page_size, hd) == BG_OK;
    if (hd == 128) return by_keys ? am_launch<128, true>(map, map5, p, n_qblk, n_splits_launch, stream)
                                  : am_launch<128, false>(map, map5, p, n_qblk, n_splits_launch, stream);
    if (hd == 64) return by_keys ? am_launch<64, true>(map, map5, p, n_qblk, n_splits_launch, stream)
                                 : am_launch<64, false>(map, map5, p, n_qblk, n_splits_launch, stream);
    return BG_ERR_UNSUPPORTED;
}
