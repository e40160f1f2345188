// out[M, N] = x[M, K] * W[N, K]^T in true 32-bit: float operands, fused
// multiply-adds on the CUDA cores, no tensor-core mode of any kind.  Each output
// element is accumulated over k in ascending order by one thread, so its value
// depends on its own row of x and row of W only: not on M, not on the tiling of
// other rows.  Any M, N, K.  Optional epilogue: cap * tanh(v / cap).
#include "common.cuh"

namespace janis {

constexpr int BM = 64, BN = 64, BK = 16;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ x, const float* __restrict__ W, float* __restrict__ out, int M, int N,
                int K, float cap) {
    __shared__ float xs[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
    grid_dependents_launch();
    grid_dependency_wait();                           // x is the kernel before's result
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 rows x 16 k of each operand: 1024 elements, 4 per thread, k fastest
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * 256;
            const int r = idx / BK, kk = idx % BK;
            const int k = k0 + kk;
            xs[kk][r] = (m0 + r < M && k < K) ? x[(size_t)(m0 + r) * K + k] : 0.f;
            ws[kk][r] = (n0 + r < N && k < K) ? W[(size_t)(n0 + r) * K + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][tm + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[kk][tn + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + tm + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tn + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (cap > 0.f) v = cap * tanhf(v / cap);
            out[(size_t)m * N + n] = v;
        }
    }
}

}  // namespace janis

using namespace janis;

JANIS_EXPORT int janis_gemm_f32(const float* x, const float* W, float* out, int M, int N, int K, float cap,
                                cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return fail("gemm_f32: K must be positive, found %d", K);
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return fail("gemm_f32: too many rows (%d)", M);
    return launch_kernel("gemm_f32", gemm_f32_kernel, grid, dim3(256), 0, stream, 1, x, W, out, M, N, K, cap);
}
