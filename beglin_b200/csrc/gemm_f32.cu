// C[M, N] (+)= A[M, K] * W[N, K]^T (+ bias[N]) in true float: CUDA-core FFMA, no tensor cores and no
// reduced-precision mode (the tensor cores have no float x float kind; their tf32 kind drops
// mantissa bits).  This is the reference's linear, y[o] = bias[o] + sum_i W[o,i] x[i] with W
// row-major [out, in] (qwen_infer.c:688-691), for a batch of rows.
//
// Every output element is summed by one thread over k = 0..K-1 in order, so a row's result does not
// depend on how many other rows the call has or where the row stands among them.
#include "common.cuh"

namespace bg {

constexpr int GF_BM = 64, GF_BN = 64, GF_BK = 16, GF_THREADS = 256;

__global__ void __launch_bounds__(GF_THREADS)
gemm_f32_nt_kernel(const float* __restrict__ A, int lda, const float* __restrict__ W, int ldw,
                   const float* __restrict__ bias, float* __restrict__ C, int ldc,
                   int M, int N, int K, int accumulate) {
    pdl_launch();
    pdl_wait();
    __shared__ float As[GF_BK][GF_BM + 4];
    __shared__ float Ws[GF_BK][GF_BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * GF_BM, n0 = blockIdx.x * GF_BN;
    const int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads, each a 4 x 4 block of C
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    // each thread loads 4 elements of A and 4 of W per k-tile: row = tid / 4, k = (tid % 4) * 4 + 0..3
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    for (int k0 = 0; k0 < K; k0 += GF_BK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            int k = k0 + lk + e;
            int am = m0 + lr, wn = n0 + lr;
            As[lk + e][lr] = (am < M && k < K) ? A[(size_t)am * lda + k] : 0.0f;
            Ws[lk + e][lr] = (wn < N && k < K) ? W[(size_t)wn * ldw + k] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GF_BK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            float* c = C + (size_t)m * ldc + n;
            *c = accumulate ? (*c + v) : v;
        }
    }
}

}  // namespace bg

extern "C" int bg_gemm_f32_nt(const float* A, int lda, const float* W, int ldw, const float* bias, float* C, int ldc,
                              int M, int N, int K, int accumulate, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return BG_OK;
    if (K <= 0) return BG_ERR_SHAPE;
    dim3 grid((N + bg::GF_BN - 1) / bg::GF_BN, (M + bg::GF_BM - 1) / bg::GF_BM);
    if (grid.y > 65535) return BG_ERR_SHAPE;
    bg::launch(bg::gemm_f32_nt_kernel, grid, dim3(bg::GF_THREADS), 0, stream, A, lda, W, ldw, bias, C, ldc, M, N, K, accumulate);
    BG_LAUNCH_CHECK();
    return BG_OK;
}
