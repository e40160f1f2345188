// Skinny bfloat16 product for decoding: out[M, N] = x[M, K] * W[N, K]^T with M <= 64
// (one row per live sequence).  The step is bound by reading W once from HBM, so W
// is the 16-row operand of mma.sync.m16n8k16 and the batch rows are the 8-wide
// operand: every weight byte is read once, whatever M is.
//
// One CTA owns 16 rows of W; its warps split K between them in blocks of 32 and
// the partial sums are added in warp order through shared memory, so a result
// does not depend on the grid.  Each thread reads 16 contiguous bytes of two rows
// of W straight into registers; the k order inside a block of 32 is permuted the
// same way for both operands, which leaves the dot product unchanged.
//
// Epilogues: none; gated activation over rows of W that alternate 8 gate rows and
// 8 up rows (one mma tile then holds matching pairs); cap * tanh(v / cap).
// Accumulation is float; the output is bfloat16 or float.  K must be a multiple of 8.
#include "common.cuh"

namespace janis {

constexpr int GEMV_WARPS = 8;

enum { EPI_NONE = 0, EPI_GATED_GELU = 1, EPI_SOFTCAP = 2, EPI_GATED_SILU = 3 };

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {   // read once: do not keep in L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

template <int MT, int U, typename TO>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
gemv_bf16_kernel(const bf16* __restrict__ x, const bf16* __restrict__ W, TO* __restrict__ out, int M, int N,
                 int K, int epi, float cap) {
    __shared__ float red[GEMV_WARPS][MT][32][4];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int r0 = blockIdx.x * 16;
    // rows past the end read the last row; their results are never stored
    const int row_lo = min(r0 + g, N - 1), row_hi = min(r0 + g + 8, N - 1);
    const bf16* wlo = W + (size_t)row_lo * K + t * 8;
    const bf16* whi = W + (size_t)row_hi * K + t * 8;
    const bf16* xr[MT];
    bool xok[MT];
#pragma unroll
    for (int i = 0; i < MT; ++i) {
        const int m = i * 8 + g;
        xok[i] = m < M;
        xr[i] = x + (size_t)min(m, M - 1) * K + t * 8;
    }
    float acc[MT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[i][c] = 0.f;

    const int nblk = (K + 31) / 32;
    for (int kb = warp; kb < nblk; kb += GEMV_WARPS * U) {
        uint4 a_lo[U], a_hi[U], b[U][MT];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k0 = (kb + u * GEMV_WARPS) * 32;
            const bool in = k0 + t * 8 < K;          // K % 8 == 0: a 16-byte piece is all in or all out
            a_lo[u] = in ? ldg_stream(wlo + k0) : make_uint4(0, 0, 0, 0);
            a_hi[u] = in ? ldg_stream(whi + k0) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int i = 0; i < MT; ++i)
                b[u][i] = (in && xok[i]) ? *reinterpret_cast<const uint4*>(xr[i] + k0) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                mma_bf16(acc[i], a_lo[u].x, a_hi[u].x, a_lo[u].y, a_hi[u].y, b[u][i].x, b[u][i].y);
                mma_bf16(acc[i], a_lo[u].z, a_hi[u].z, a_lo[u].w, a_hi[u].w, b[u][i].z, b[u][i].w);
            }
    }
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) red[warp][i][lane][c] = acc[i][c];
    __syncthreads();

    if (epi == EPI_GATED_GELU || epi == EPI_GATED_SILU) {
        // rows g of the tile are gate rows, rows g + 8 the matching up rows
        const int I = N / 2;
        for (int idx = threadIdx.x; idx < MT * 32 * 2; idx += blockDim.x) {
            const int i = idx / 64, ln = (idx / 2) % 32, p = idx % 2;
            float gate = 0.f, up = 0.f;
#pragma unroll
            for (int w = 0; w < GEMV_WARPS; ++w) {
                gate += red[w][i][ln][p];
                up += red[w][i][ln][p + 2];
            }
            const int m = i * 8 + (ln & 3) * 2 + p;
            const int j = blockIdx.x * 8 + (ln >> 2);
            if (m < M && j < I) {
                const float a = epi == EPI_GATED_GELU ? gelu_tanh(gate) : gate / (1.0f + expf(-gate));
                out[(size_t)m * I + j] = from_float<TO>(a * up);
            }
        }
        return;
    }
    for (int idx = threadIdx.x; idx < MT * 32 * 4; idx += blockDim.x) {
        const int i = idx / 128, ln = (idx / 4) % 32, c = idx % 4;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < GEMV_WARPS; ++w) v += red[w][i][ln][c];
        const int m = i * 8 + (ln & 3) * 2 + (c & 1);
        const int n = r0 + (ln >> 2) + (c >> 1) * 8;
        if (m < M && n < N) {
            if (epi == EPI_SOFTCAP && cap > 0.f) v = cap * tanhf(v / cap);
            out[(size_t)m * N + n] = from_float<TO>(v);
        }
    }
}

}  // namespace janis

using namespace janis;

template <int MT, int U>
static int launch_gemv(const bf16* x, const bf16* W, void* out, int out_dtype, int M, int N, int K, int epi,
                       float cap, cudaStream_t stream) {
    const int grid = (N + 15) / 16;
    if (out_dtype == JANIS_BF16)
        gemv_bf16_kernel<MT, U, bf16><<<grid, GEMV_WARPS * 32, 0, stream>>>(x, W, (bf16*)out, M, N, K, epi, cap);
    else
        gemv_bf16_kernel<MT, U, float><<<grid, GEMV_WARPS * 32, 0, stream>>>(x, W, (float*)out, M, N, K, epi, cap);
    return launched("gemv_bf16");
}

// x [M, K] bf16, W [N, K] bf16, out [M, N] (or [M, N/2] with a gated epilogue)
JANIS_EXPORT int janis_gemv_bf16(const void* x, const void* W, void* out, int out_dtype, int M, int N, int K,
                                 int epi, float cap, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64) return fail("gemv_bf16: at most 64 rows, found %d", M);
    if (K <= 0 || K % 8) return fail("gemv_bf16: K must be a positive multiple of 8, found %d", K);
    if (out_dtype != JANIS_BF16 && out_dtype != JANIS_F32) return fail("gemv_bf16: unknown output dtype %d", out_dtype);
    if ((epi == EPI_GATED_GELU || epi == EPI_GATED_SILU) && N % 16)
        return fail("gemv_bf16: a gated epilogue needs N to be a multiple of 16, found %d", N);
    if (epi < 0 || epi > 3) return fail("gemv_bf16: unknown epilogue %d", epi);
    if (((uintptr_t)x | (uintptr_t)W) & 15) return fail("gemv_bf16: operands must be 16-byte aligned");
    const bf16* xp = (const bf16*)x;
    const bf16* wp = (const bf16*)W;
    if (M <= 8) return launch_gemv<1, 4>(xp, wp, out, out_dtype, M, N, K, epi, cap, stream);
    if (M <= 16) return launch_gemv<2, 4>(xp, wp, out, out_dtype, M, N, K, epi, cap, stream);
    if (M <= 32) return launch_gemv<4, 2>(xp, wp, out, out_dtype, M, N, K, epi, cap, stream);
    return launch_gemv<8, 1>(xp, wp, out, out_dtype, M, N, K, epi, cap, stream);
}
