// Shared helpers of the sm_100a kernels: element types, loads and stores that convert to and
// from float, warp and block reductions, and the status word in which a kernel records a bad
// index instead of touching memory it does not own.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define BG_DTYPE_F32 0
#define BG_DTYPE_BF16 1

// Return codes of the extern "C" entry points: 0 is success, a positive value is a cudaError_t,
// a negative one says which argument was refused.
#define BG_OK 0
#define BG_ERR_DTYPE (-1)
#define BG_ERR_SHAPE (-2)
#define BG_ERR_ALIGN (-3)
#define BG_ERR_UNSUPPORTED (-4)

// Bits of the device status word.
#define BG_STATUS_BAD_TOKEN 1u      // a token id outside [0, vocab)
#define BG_STATUS_BAD_PAGE 2u       // a block-table entry outside [0, num_pages)
#define BG_STATUS_TIMEOUT 4u        // a bounded wait ran out

// Dynamic shared memory from which a kernel asks for more than the default: the default limit of 48 KB holds for
// a kernel's static and dynamic shared memory together, so a request of exactly 48 KB beside a few static
// words is refused at launch unless the larger limit was asked for.
#define BG_SMEM_OPT_IN (40 * 1024)

#define BG_LAUNCH_CHECK() \
    do { cudaError_t e_ = cudaGetLastError(); if (e_ != cudaSuccess) return (int)e_; } while (0)

namespace bg {

// Programmatic dependent launch: a kernel launched with the attribute below may begin (be scheduled,
// set up shared memory, fetch what no earlier kernel of the step writes, such as weights) while its
// predecessor in the stream is still running.  It must call pdl_wait() before it reads anything an
// earlier kernel wrote and before it writes global memory; pdl_wait returns once the predecessor has
// completed and its writes are visible.  Every kernel of this library calls pdl_launch() first (its
// successor may be scheduled as soon as all of this grid's blocks run) and pdl_wait() before it
// touches the step's data, so completion carries along the chain.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

#ifdef __CUDACC__
// 1: launch with the programmatic-serialization attribute (default); 0: plain launches.
inline int& pdl_enabled() {
    static int on = [] { const char* e = getenv("BEGLIN_B200_PDL"); return (e && e[0] == '0') ? 0 : 1; }();
    return on;
}

// The number of SMs of the current device, read from the device once per device.
inline int sm_count() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
        cached[dev] = n;
    }
    return cached[dev];
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// The same for a kernel whose CTAs form thread block clusters of (1, 1, cluster_z).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_cluster(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster_z,
                                  Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1; attr[n].val.clusterDim.y = 1; attr[n].val.clusterDim.z = (unsigned)cluster_z;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}
#endif

// Keys per split of a request's keys.  A positive `split` is taken as it is (the same boundaries for every
// request: results then do not depend on a request's length).  split <= 0 spreads the request's own
// n_keys evenly over the n_splits CTAs that the grid has for it, in multiples of 256 (decoding inside a
// captured graph, whose grid is fixed while the requests grow).
__host__ __device__ __forceinline__ int keys_per_split(int split, int n_keys, int n_splits) {
    if (split > 0) return split;
    const int s = (n_keys + n_splits - 1) / n_splits;
    const int r = (s + 255) / 256 * 256;
    return r < 256 ? 256 : r;
}

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Thread block clusters: the cluster-wide barrier (every thread of every CTA arrives) and stores into a
// peer CTA's shared memory.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory"); }
// (nothing that this thread wrote has to be visible to the peers at the first use of the barrier)
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_sync_all() {
    cluster_arrive();
    cluster_wait();
}
// the address, in the cluster's shared window, of this CTA's shared-memory address in the CTA of the given rank
__device__ __forceinline__ unsigned peer_addr(unsigned local_addr, unsigned rank) {
    unsigned a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(a) : "r"(local_addr), "r"(rank));
    return a;
}
__device__ __forceinline__ void st_cluster(unsigned addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(addr), "f"(v) : "memory");
}
// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? scratch[lane] : 0.0f;
    t = warp_sum(t);
    return t;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    return t;
}

// Eight consecutive values as floats, from 16-byte aligned memory, and back.
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
    uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
}

// Sum of `parts` float4 values that lie `stride4` float4 apart, added in index order.  For up to sixteen parts the
// count picks a branch with exactly that many loads and no condition among them, so that they all go out together
// and the sum costs one round trip (with a condition on every load the compiler kept few of them in flight: the
// norm over 5 partial sums of 32 rows of 3,584 took 3.9 us that way and 3.5 us this way).
template <int N>
__device__ __forceinline__ float4 sum_parts4_of(const float4* p, size_t stride4) {
    float4 a[N];
#pragma unroll
    for (int j = 0; j < N; ++j) a[j] = p[(size_t)j * stride4];
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (int j = 0; j < N; ++j) { acc.x += a[j].x; acc.y += a[j].y; acc.z += a[j].z; acc.w += a[j].w; }
    return acc;
}
__device__ __forceinline__ float4 sum_parts4(const float4* p, int parts, size_t stride4) {
    switch (parts) {
        case 1: return sum_parts4_of<1>(p, stride4);
        case 2: return sum_parts4_of<2>(p, stride4);
        case 3: return sum_parts4_of<3>(p, stride4);
        case 4: return sum_parts4_of<4>(p, stride4);
        case 5: return sum_parts4_of<5>(p, stride4);
        case 6: return sum_parts4_of<6>(p, stride4);
        case 7: return sum_parts4_of<7>(p, stride4);
        case 8: return sum_parts4_of<8>(p, stride4);
        case 9: return sum_parts4_of<9>(p, stride4);
        case 10: return sum_parts4_of<10>(p, stride4);
        case 11: return sum_parts4_of<11>(p, stride4);
        case 12: return sum_parts4_of<12>(p, stride4);
        case 13: return sum_parts4_of<13>(p, stride4);
        case 14: return sum_parts4_of<14>(p, stride4);
        case 15: return sum_parts4_of<15>(p, stride4);
        case 16: return sum_parts4_of<16>(p, stride4);
        default: break;
    }
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int p0 = 0; p0 < parts; p0 += 16) {
        float4 a[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) a[j] = (p0 + j < parts) ? p[(size_t)(p0 + j) * stride4] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int j = 0; j < 16; ++j) { acc.x += a[j].x; acc.y += a[j].y; acc.z += a[j].z; acc.w += a[j].w; }
    }
    return acc;
}
// The same for single values of any element type.
template <typename T>
__device__ __forceinline__ float sum_parts(const T* p, int parts, size_t stride) {
    float acc = 0.0f;
    for (int p0 = 0; p0 < parts; p0 += 8) {
        float a[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = (p0 + j < parts) ? to_float(p[(size_t)(p0 + j) * stride]) : 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc += a[j];
    }
    return acc;
}

}  // namespace bg

// Dispatch on a runtime dtype code to a template argument.
#define BG_DISPATCH_DTYPE(code, T, ...)                                   \
    do {                                                                  \
        if ((code) == BG_DTYPE_F32) { using T = float; __VA_ARGS__; }     \
        else if ((code) == BG_DTYPE_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
        else return BG_ERR_DTYPE;                                         \
    } while (0)
