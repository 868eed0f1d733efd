// Grouped-query attention over the paged cache, for prompt portions and decoded tokens alike.
//
// A step's token rows are cut into query blocks: up to `bq` consecutive rows of ONE request.  The
// keys are cut into splits of `split` positions at absolute boundaries (0, split, 2*split, ...).
// One CTA takes (query block, kv head, split): it streams that split's keys and values once for all
// query heads of the group (the reference's per-KV-group variant, attn_neon.h:130-175) and keeps,
// for every (row, head), a running maximum, a running sum and an unnormalised output.  It writes
// them as a partial result; `attention_merge` joins the partials of a row in split order.
//
// The math of one (row, head) is that of qwen_infer.c:1538-1543: s_t = (q . K_t) * scale for the
// visible t (t <= position, and t > position - window when there is a window), softmax with the
// maximum subtracted, o = sum_t p_t V_t.  Everything is float.  Because tiles and splits start at
// absolute positions and a row never shares an accumulator with another row, the result of a row
// does not depend on how the step was cut or on what else is in the batch.
#include "common.cuh"

namespace bg {

constexpr int ATT_THREADS = 256;
constexpr int ATT_WARPS = ATT_THREADS / 32;
constexpr int ATT_MAX_DPL = 8;      // head_dim <= 256: at most 8 output features per lane

struct AttnParams {
    const void* q;          // [T, nh, hd] with row stride q_stride (elements)
    int q_stride;
    const void* kv_pool;    // [num_pages][2][nkv][page_size][hd]
    int num_pages, page_size;
    const int* block_table; // [B, max_pages]
    int max_pages;
    const int* positions;   // [T]
    const int* qblk;        // [n_qblk][3] = (request, first row, number of rows)
    float* part_o;          // [T*nh][max_splits][hd]
    float* part_ml;         // [T*nh][max_splits][2]
    int max_splits;
    int nh, nkv, hd, group;
    int window;             // 0: none
    int split;              // keys per split
    int tile;               // keys per shared-memory tile (32 or 64), divides split
    int bq;                 // rows per query block (upper bound)
    float scale;
    unsigned* status;
};

template <typename TQ, typename TC>
__global__ void __launch_bounds__(ATT_THREADS)
attention_partial_kernel(AttnParams p) {
    extern __shared__ float smem[];
    const int hd = p.hd, group = p.group;
    const int kstride = hd + 1;
    const int n_rows_max = p.bq * group;
    float* q_s = smem;                                   // [n_rows_max][hd]
    float* acc_s = q_s + (size_t)n_rows_max * hd;        // [n_rows_max][hd]
    float* k_s = acc_s + (size_t)n_rows_max * hd;        // [tile][hd+1]
    float* v_s = k_s + (size_t)p.tile * kstride;         // [tile][hd]
    float* m_s = v_s + (size_t)p.tile * hd;              // [n_rows_max]
    float* l_s = m_s + n_rows_max;                       // [n_rows_max]
    long long* base_s = (long long*)(l_s + n_rows_max);   // [tile] element offsets (the float count before it is even)

    pdl_launch();
    pdl_wait();
    const int qb = blockIdx.x, kvh = blockIdx.y, sp = blockIdx.z;
    const int req = p.qblk[qb * 3 + 0], row0 = p.qblk[qb * 3 + 1], nq = p.qblk[qb * 3 + 2];
    if (nq <= 0) return;
    const int pos_first = p.positions[row0];
    const int pos_last = p.positions[row0 + nq - 1];
    const int lo_first = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
    const int k_begin = max(sp * p.split, lo_first);
    const int k_end = min((sp + 1) * p.split, pos_last + 1);       // exclusive
    if (k_begin >= k_end) return;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_rows = nq * group;
    const TQ* q = (const TQ*)p.q;
    for (int idx = tid; idx < n_rows * hd; idx += ATT_THREADS) {
        int r = idx / hd, d = idx - r * hd;
        int qi = r / group, g = r - qi * group;
        q_s[idx] = to_float(q[(size_t)(row0 + qi) * p.q_stride + (size_t)(kvh * group + g) * hd + d]);
        acc_s[idx] = 0.0f;
    }
    for (int r = tid; r < n_rows; r += ATT_THREADS) { m_s[r] = -INFINITY; l_s[r] = 0.0f; }

    const TC* pool = (const TC*)p.kv_pool;
    const size_t page_elems = (size_t)2 * p.nkv * p.page_size * hd;
    const size_t v_off = (size_t)p.nkv * p.page_size * hd;
    const int tile = p.tile;
    const int t_first = (k_begin / tile) * tile;

    for (int t0 = t_first; t0 < k_end; t0 += tile) {
        __syncthreads();
        // element offset of each key's K row in the pool, or -1 for a key outside [k_begin, k_end)
        for (int j = tid; j < tile; j += ATT_THREADS) {
            int key = t0 + j;
            long long off = -1;
            if (key >= k_begin && key < k_end) {
                int page = p.block_table[(size_t)req * p.max_pages + key / p.page_size];
                if (page < 0 || page >= p.num_pages) {
                    if (p.status) atomicOr(p.status, BG_STATUS_BAD_PAGE);
                } else {
                    off = (long long)((size_t)page * page_elems + ((size_t)kvh * p.page_size + key % p.page_size) * hd);
                }
            }
            base_s[j] = off;
        }
        __syncthreads();
        for (int idx = tid; idx < tile * hd; idx += ATT_THREADS) {
            int j = idx / hd, d = idx - j * hd;
            long long off = base_s[j];
            float kv = 0.0f, vv = 0.0f;
            if (off >= 0) { kv = to_float(pool[off + d]); vv = to_float(pool[off + v_off + d]); }
            k_s[j * kstride + d] = kv;
            v_s[j * hd + d] = vv;
        }
        __syncthreads();

        for (int r = warp; r < n_rows; r += ATT_WARPS) {
            const int qi = r / group;
            const int pos = p.positions[row0 + qi];
            const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
            const float* qr = q_s + (size_t)r * hd;
            float s[2];
            float tmax = -INFINITY;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                s[c] = -INFINITY;
                int j = c * 32 + lane;
                if (j < tile) {
                    int key = t0 + j;
                    if (key >= lo && key <= pos && key >= k_begin && key < k_end && base_s[j] >= 0) {
                        const float* kr = k_s + j * kstride;
                        float dot = 0.0f;
                        for (int d = 0; d < hd; ++d) dot = fmaf(qr[d], kr[d], dot);
                        s[c] = dot * p.scale;
                    }
                }
                tmax = fmaxf(tmax, s[c]);
            }
            tmax = warp_max(tmax);
            if (tmax == -INFINITY) continue;            // no visible key of this tile for this row
            const float m_old = m_s[r];
            const float m_new = fmaxf(m_old, tmax);
            const float corr = (m_old == -INFINITY) ? 0.0f : expf(m_old - m_new);
            float psum = 0.0f;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                s[c] = (s[c] == -INFINITY) ? 0.0f : expf(s[c] - m_new);
                psum += s[c];
            }
            psum = warp_sum(psum);
            float acc[ATT_MAX_DPL];
            float* ar = acc_s + (size_t)r * hd;
#pragma unroll
            for (int i = 0; i < ATT_MAX_DPL; ++i) {
                int d = i * 32 + lane;
                acc[i] = (d < hd) ? ar[d] * corr : 0.0f;
            }
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                if (c * 32 >= tile) break;
                for (int jj = 0; jj < 32; ++jj) {
                    float pj = __shfl_sync(0xffffffffu, s[c], jj);
                    if (pj != 0.0f) {
                        const float* vr = v_s + (c * 32 + jj) * hd;
#pragma unroll
                        for (int i = 0; i < ATT_MAX_DPL; ++i) {
                            int d = i * 32 + lane;
                            if (d < hd) acc[i] = fmaf(pj, vr[d], acc[i]);
                        }
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < ATT_MAX_DPL; ++i) {
                int d = i * 32 + lane;
                if (d < hd) ar[d] = acc[i];
            }
            if (lane == 0) { m_s[r] = m_new; l_s[r] = l_s[r] * corr + psum; }
        }
    }
    __syncthreads();
    // partial results, only for rows that see at least one key of this split
    for (int r = warp; r < n_rows; r += ATT_WARPS) {
        const int qi = r / group, g = r - qi * group;
        const int pos = p.positions[row0 + qi];
        const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
        if (pos < sp * p.split || lo >= (sp + 1) * p.split) continue;
        const size_t prow = ((size_t)(row0 + qi) * p.nh + (size_t)kvh * group + g) * p.max_splits + sp;
        for (int d = lane; d < hd; d += 32) p.part_o[prow * hd + d] = acc_s[(size_t)r * hd + d];
        if (lane == 0) { p.part_ml[prow * 2 + 0] = m_s[r]; p.part_ml[prow * 2 + 1] = l_s[r]; }
    }
}

// out[t, h, :] = sum_s o_s * exp(m_s - m) / sum_s l_s * exp(m_s - m), over the splits the row sees,
// in split order.  One warp per (row, head): the lanes first take one split each (of up to 32 * MERGE_GROUPS
// at once) to find the maximum and the weights, so these loads are in flight together and are made once; then
// every lane sums its output features over the splits, BATCH splits' loads on their way at a time.  DPL is the
// number of output features per lane (head_dim <= 32 DPL).
constexpr int MERGE_GROUPS = 4;
template <typename TO, int DPL, int BATCH>
__global__ void attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                       const int* __restrict__ positions, TO* __restrict__ out, int out_stride,
                                       int T, int nh, int hd, int max_splits, int split_arg, int window) {
    pdl_launch();
    pdl_wait();
    const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= T * nh) return;
    const int t = w / nh, h = w - t * nh;
    const int pos = positions[t];
    const int split = keys_per_split(split_arg, pos + 1, max_splits);
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int s_lo = lo / split, s_hi = pos / split;
    const size_t prow = (size_t)w * max_splits;
    // the maxima and sums of the first 32 * MERGE_GROUPS splits of the row: lane j holds split s_lo + 32 g + j
    float ms_r[MERGE_GROUPS], ls_r[MERGE_GROUPS];
#pragma unroll
    for (int g = 0; g < MERGE_GROUPS; ++g) {
        const int sidx = s_lo + 32 * g + lane;
        const float2 ml = sidx <= s_hi ? *reinterpret_cast<const float2*>(part_ml + (prow + sidx) * 2) : make_float2(-INFINITY, 0.0f);
        ms_r[g] = ml.x; ls_r[g] = ml.y;
    }
    float m = -INFINITY;
#pragma unroll
    for (int g = 0; g < MERGE_GROUPS; ++g) m = fmaxf(m, ms_r[g]);
    for (int sidx = s_lo + 32 * MERGE_GROUPS + lane; sidx <= s_hi; sidx += 32) m = fmaxf(m, part_ml[(prow + sidx) * 2]);
    m = warp_max(m);
    float acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] = 0.0f;
    float l = 0.0f;
    int grp = 0;
    for (int s0 = s_lo; s0 <= s_hi; s0 += 32, ++grp) {
        // this lane's split of the group of 32: its weight and its share of the sum
        const int mine = s0 + lane;
        float ms = -INFINITY, l_mine = 0.0f;
        if (grp < MERGE_GROUPS) {
#pragma unroll
            for (int g = 0; g < MERGE_GROUPS; ++g) if (g == grp) { ms = ms_r[g]; l_mine = ls_r[g]; }
        } else if (mine <= s_hi) {
            ms = part_ml[(prow + mine) * 2];
            l_mine = part_ml[(prow + mine) * 2 + 1];
        }
        const float f_mine = (ms == -INFINITY) ? 0.0f : expf(ms - m);
        const int n = min(32, s_hi - s0 + 1);
        for (int j0 = 0; j0 < n; j0 += BATCH) {
            // the loads of BATCH splits go out together, then they are added in split order
            float v[BATCH][DPL];
#pragma unroll
            for (int jj = 0; jj < BATCH; ++jj) {
                const float* po = part_o + (prow + s0 + j0 + jj) * hd;
#pragma unroll
                for (int i = 0; i < DPL; ++i) {
                    int d = i * 32 + lane;
                    v[jj][i] = (j0 + jj < n && d < hd) ? po[d] : 0.0f;
                }
            }
#pragma unroll
            for (int jj = 0; jj < BATCH; ++jj) {
                const float f = __shfl_sync(0xffffffffu, f_mine, (j0 + jj) & 31);
                const float lj = __shfl_sync(0xffffffffu, l_mine, (j0 + jj) & 31);
                if (j0 + jj < n) {
                    l = fmaf(lj, f, l);
#pragma unroll
                    for (int i = 0; i < DPL; ++i) acc[i] = fmaf(v[jj][i], f, acc[i]);
                }
            }
        }
    }
    const float inv = 1.0f / l;
    TO* o = out + (size_t)t * out_stride + (size_t)h * hd;
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
        int d = i * 32 + lane;
        if (d < hd) o[d] = from_float<TO>(acc[i] * inv);
    }
}

}  // namespace bg

using namespace bg;

static size_t attention_smem_bytes(int bq, int group, int hd, int tile) {
    size_t rows = (size_t)bq * group;
    size_t floats = rows * hd * 2 + (size_t)tile * (hd + 1) + (size_t)tile * hd + rows * 2;
    return floats * sizeof(float) + (size_t)tile * sizeof(long long) + 8;
}

// Rows per query block and keys per tile that fit the shared memory of one CTA for these sizes.
// Returns 0 and fills bq and tile, or BG_ERR_UNSUPPORTED.
extern "C" int bg_attention_plan(int group, int hd, int* bq_out, int* tile_out) {
    if (hd <= 0 || hd > 32 * ATT_MAX_DPL || group <= 0) return BG_ERR_UNSUPPORTED;
    const size_t limit = 200 * 1024;
    for (int tile = 64; tile >= 32; tile >>= 1) {
        for (int bq = 16; bq >= 1; bq >>= 1) {
            if (attention_smem_bytes(bq, group, hd, tile) <= limit) { *bq_out = bq; *tile_out = tile; return BG_OK; }
        }
    }
    return BG_ERR_UNSUPPORTED;
}

extern "C" int bg_attention_partial(const void* q, int q_dtype, int q_stride, const void* kv_pool, int cache_dtype,
                                    int num_pages, int page_size, const int* block_table, int max_pages,
                                    const int* positions, const int* qblk, int n_qblk, float* part_o, float* part_ml,
                                    int max_splits, int n_splits_launch, int nh, int nkv, int hd, int window, int split,
                                    int tile, int bq, float scale, unsigned* status, cudaStream_t stream) {
    if (n_qblk <= 0 || n_splits_launch <= 0) return BG_OK;
    if (nh % nkv != 0 || hd > 32 * ATT_MAX_DPL || (tile != 32 && tile != 64) || split % tile != 0) return BG_ERR_SHAPE;
    if (n_splits_launch > max_splits || n_splits_launch > 65535 || nkv > 65535) return BG_ERR_SHAPE;
    AttnParams p;
    p.q = q; p.q_stride = q_stride; p.kv_pool = kv_pool; p.num_pages = num_pages; p.page_size = page_size;
    p.block_table = block_table; p.max_pages = max_pages; p.positions = positions; p.qblk = qblk;
    p.part_o = part_o; p.part_ml = part_ml; p.max_splits = max_splits; p.nh = nh; p.nkv = nkv; p.hd = hd;
    p.group = nh / nkv; p.window = window; p.split = split; p.tile = tile; p.bq = bq; p.scale = scale; p.status = status;
    size_t smem = attention_smem_bytes(bq, p.group, hd, tile);
    if (smem > 227 * 1024) return BG_ERR_UNSUPPORTED;
    dim3 grid(n_qblk, nkv, n_splits_launch);
#define BG_ATT_LAUNCH(TQ, TC)                                                                              \
    do {                                                                                                   \
        auto kern = attention_partial_kernel<TQ, TC>;                                                      \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) return (int)e;                                                               \
        launch(kern, grid, dim3(ATT_THREADS), smem, stream, p);                                                      \
    } while (0)
    if (q_dtype == BG_DTYPE_F32 && cache_dtype == BG_DTYPE_F32) BG_ATT_LAUNCH(float, float);
    else if (q_dtype == BG_DTYPE_BF16 && cache_dtype == BG_DTYPE_BF16) BG_ATT_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (q_dtype == BG_DTYPE_F32 && cache_dtype == BG_DTYPE_BF16) BG_ATT_LAUNCH(float, __nv_bfloat16);
    else if (q_dtype == BG_DTYPE_BF16 && cache_dtype == BG_DTYPE_F32) BG_ATT_LAUNCH(__nv_bfloat16, float);
    else return BG_ERR_DTYPE;
#undef BG_ATT_LAUNCH
    BG_LAUNCH_CHECK();
    return BG_OK;
}

// The same for at most NS (8 or 16) splits and head_dim <= 128 (decoding): the maxima and sums and the partial outputs
// of ALL splits are asked for at once, and what lies outside the row's range is dropped, so the kernel is one round
// trip to memory instead of three.  The row's range of splits comes from its position alone, which no kernel of the
// step writes: it is worked out before the wait for the kernel ahead.
template <typename TO, int NS>
__global__ void attention_merge_few_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                           const int* __restrict__ positions, TO* __restrict__ out, int out_stride,
                                           int T, int nh, int hd, int max_splits, int split_arg, int window) {
    pdl_launch();
    const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const bool idle = w >= T * nh;
    const int t = idle ? 0 : w / nh, h = w - t * nh;
    const size_t prow = (size_t)w * max_splits;
    // the row's position is written by no kernel of the step: its range of splits (three integer divisions) is
    // worked out while the kernel ahead still runs
    const int pos = positions[t];
    const int split = keys_per_split(split_arg, pos + 1, max_splits);
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int s_lo = lo / split, s_hi = pos / split;
    pdl_wait();
    if (idle) return;                  // (not before the wait: with warps of a CTA gone before it, rows came out wrong)
    float ms[NS], ls[NS], v[NS][4];
#pragma unroll
    for (int s = 0; s < NS; ++s) {
        const bool have = s < max_splits;
        ms[s] = have ? part_ml[(prow + s) * 2] : -INFINITY;
        ls[s] = have ? part_ml[(prow + s) * 2 + 1] : 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int d = i * 32 + lane;
            v[s][i] = (have && d < hd) ? part_o[(prow + s) * hd + d] : 0.0f;
        }
    }
    float m = -INFINITY;
#pragma unroll
    for (int s = 0; s < NS; ++s) {
        if (s < s_lo || s > s_hi) ms[s] = -INFINITY;          // not written for this row: whatever was read is dropped
        m = fmaxf(m, ms[s]);
    }
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, l = 0.0f;
#pragma unroll
    for (int s = 0; s < NS; ++s) {                             // in split order
        if (ms[s] != -INFINITY) {
            const float f = expf(ms[s] - m);
            l = fmaf(ls[s], f, l);
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[i] = fmaf(v[s][i], f, acc[i]);
        }
    }
    const float inv = 1.0f / l;
    TO* o = out + (size_t)t * out_stride + (size_t)h * hd;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int d = i * 32 + lane;
        if (d < hd) o[d] = from_float<TO>(acc[i] * inv);
    }
}

// The same for many splits of few rows (decoding a long context at a small batch, where a request's keys are
// spread over up to a whole wave of CTAs): a CTA of eight warps per (row, head).  The splits are taken in groups
// of eight consecutive ABSOLUTE split numbers; warp w owns the groups w, w + 8, ...: it asks for the eight partial
// outputs of a group at once (a lane holds four features), joins them in split order around the group's own
// maximum, and joins its groups in ascending order; the eight warps' results are joined in warp order through
// shared memory.  The grouping depends on the split numbers alone, so a row's result depends on nothing but its
// own range of splits.  One trip to memory per group instead of one per 16 splits of a single warp.
constexpr int MERGE_WARPS = 8;
template <typename TO>
__global__ void __launch_bounds__(32 * MERGE_WARPS)
attention_merge_block_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                             const int* __restrict__ positions, TO* __restrict__ out, int out_stride,
                             int T, int nh, int hd, int max_splits, int split_arg, int window) {
    __shared__ float4 acc_s[MERGE_WARPS][32];
    __shared__ float2 ml_s[MERGE_WARPS];
    pdl_launch();
    const int w = blockIdx.x;                                   // (row, head)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = w / nh, h = w - t * nh;
    // (the row's position is written by no kernel of the step: its range of splits is worked out before the wait)
    const int pos = positions[t];
    const int split = keys_per_split(split_arg, pos + 1, max_splits);
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int s_lo = lo / split, s_hi = pos / split;
    pdl_wait();
    const size_t prow = (size_t)w * max_splits;
    const int d = lane * 4;
    const bool live = d < hd;                                   // hd is a multiple of 4
    float m = -INFINITY, l = 0.0f;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int g = (s_lo >> 3) + ((warp - (s_lo >> 3)) & (MERGE_WARPS - 1)); g * 8 <= s_hi; g += MERGE_WARPS) {
        float ms[8], ls[8];
        float4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int sidx = g * 8 + j;
            const bool have = sidx >= s_lo && sidx <= s_hi;
            const float2 ml = have ? *reinterpret_cast<const float2*>(part_ml + (prow + sidx) * 2) : make_float2(-INFINITY, 0.0f);
            ms[j] = ml.x; ls[j] = ml.y;
            v[j] = (have && live) ? *reinterpret_cast<const float4*>(part_o + (prow + sidx) * hd + d)
                                  : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
        float mg = -INFINITY;
#pragma unroll
        for (int j = 0; j < 8; ++j) mg = fmaxf(mg, ms[j]);
        if (mg == -INFINITY) continue;
        float lg = 0.0f;
        float4 ag = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int j = 0; j < 8; ++j) {                           // in split order
            if (ms[j] != -INFINITY) {
                const float f = expf(ms[j] - mg);
                lg = fmaf(ls[j], f, lg);
                ag.x = fmaf(v[j].x, f, ag.x); ag.y = fmaf(v[j].y, f, ag.y);
                ag.z = fmaf(v[j].z, f, ag.z); ag.w = fmaf(v[j].w, f, ag.w);
            }
        }
        const float mn = fmaxf(m, mg);
        const float fo = (m == -INFINITY) ? 0.0f : expf(m - mn), fg = expf(mg - mn);
        l = l * fo + lg * fg;
        acc.x = acc.x * fo + ag.x * fg; acc.y = acc.y * fo + ag.y * fg;
        acc.z = acc.z * fo + ag.z * fg; acc.w = acc.w * fo + ag.w * fg;
        m = mn;
    }
    acc_s[warp][lane] = acc;
    if (lane == 0) ml_s[warp] = make_float2(m, l);
    __syncthreads();
    if (warp != 0) return;
    float mt = -INFINITY;
#pragma unroll
    for (int i = 0; i < MERGE_WARPS; ++i) mt = fmaxf(mt, ml_s[i].x);
    float lt = 0.0f;
    float4 at = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (int i = 0; i < MERGE_WARPS; ++i) {                     // in warp order
        const float2 ml = ml_s[i];
        if (ml.x != -INFINITY) {
            const float f = expf(ml.x - mt);
            const float4 a = acc_s[i][lane];
            lt = fmaf(ml.y, f, lt);
            at.x = fmaf(a.x, f, at.x); at.y = fmaf(a.y, f, at.y); at.z = fmaf(a.z, f, at.z); at.w = fmaf(a.w, f, at.w);
        }
    }
    if (!live) return;
    const float inv = 1.0f / lt;
    TO* o = out + (size_t)t * out_stride + (size_t)h * hd + d;
    o[0] = from_float<TO>(at.x * inv); o[1] = from_float<TO>(at.y * inv);
    o[2] = from_float<TO>(at.z * inv); o[3] = from_float<TO>(at.w * inv);
}

extern "C" int bg_attention_merge(const float* part_o, const float* part_ml, const int* positions, void* out,
                                  int out_dtype, int out_stride, int T, int nh, int hd, int max_splits, int split,
                                  int window, cudaStream_t stream) {
    if (T <= 0) return BG_OK;
    long long warps = (long long)T * nh;
    unsigned blocks = (unsigned)((warps * 32 + 255) / 256);
    // few rows: a warp per block, so that the rows' loads go out from as many SMs as there are rows and heads
    const bool spread = warps <= 592;
    const unsigned few_blocks = spread ? (unsigned)warps : blocks, few_threads = spread ? 32u : 256u;
    const bool block_fits = hd <= 128 && hd % 4 == 0 && out_dtype == BG_DTYPE_BF16 && warps <= 4096;
    if (max_splits > 8 && warps <= 128 && block_fits) {
        // few bfloat16 rows with more than eight splits each (one or two requests): a CTA per (row, head) spreads the
        // loads over as many SMs as there are rows and heads; a warp per (row, head) keeps them on one or two
        // (one request at 4,096 positions, 16 splits: the merge cost its step 5.7 us a layer that way and 2.5 to
        // 5 us this way; the decode step of the 1.5B sizes went from 1.372 to 1.214 ms at batch 1, from 1.225 to
        // 1.151 ms at batch 2)
        launch(attention_merge_block_kernel<__nv_bfloat16>, dim3((unsigned)warps), dim3(32 * MERGE_WARPS), 0, stream,
               part_o, part_ml, positions, (__nv_bfloat16*)out, out_stride, T, nh, hd, max_splits, split, window);
    } else if (max_splits <= 8 && hd <= 128) {
        BG_DISPATCH_DTYPE(out_dtype, TO, launch(attention_merge_few_kernel<TO, 8>, dim3(few_blocks), dim3(few_threads), 0, stream,
            part_o, part_ml, positions, (TO*)out, out_stride, T, nh, hd, max_splits, split, window));
    } else if (max_splits <= 16 && hd <= 128) {
        BG_DISPATCH_DTYPE(out_dtype, TO, launch(attention_merge_few_kernel<TO, 16>, dim3(few_blocks), dim3(few_threads), 0, stream,
            part_o, part_ml, positions, (TO*)out, out_stride, T, nh, hd, max_splits, split, window));
    } else if (block_fits) {
        // bfloat16 rows of few requests with many splits each (the float path keeps one order of summation for
        // every shape of a step, so that its rows do not depend on the batch)
        launch(attention_merge_block_kernel<__nv_bfloat16>, dim3((unsigned)warps), dim3(32 * MERGE_WARPS), 0, stream,
               part_o, part_ml, positions, (__nv_bfloat16*)out, out_stride, T, nh, hd, max_splits, split, window);
    } else if (hd <= 128) {
        BG_DISPATCH_DTYPE(out_dtype, TO, launch(attention_merge_kernel<TO, 4, 16>, dim3(blocks), dim3(256), 0, stream,
            part_o, part_ml, positions, (TO*)out, out_stride, T, nh, hd, max_splits, split, window));
    } else {
        BG_DISPATCH_DTYPE(out_dtype, TO, launch(attention_merge_kernel<TO, ATT_MAX_DPL, 4>, dim3(blocks), dim3(256), 0, stream,
            part_o, part_ml, positions, (TO*)out, out_stride, T, nh, hd, max_splits, split, window));
    }
    BG_LAUNCH_CHECK();
    return BG_OK;
}
