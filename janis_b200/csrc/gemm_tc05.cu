// Skinny bfloat16 product on the 5th-generation tensor cores: out[M, N] = x[M, K] * W[N, K]^T for
// 16 < M <= 64 rows (decode steps of larger batches), bound by streaming W from HBM once.
//
// The operands are swapped: 128 rows of W are the M side of tcgen05.mma (one row per TMEM lane), the
// batch rows, padded to a multiple of 16, are its N side, so one instruction multiplies a [128 x 16]
// slice of W with all batch rows and the accumulator [128 x Mpad] float lives in tensor memory.
//   * TMA (cp.async.bulk.tensor, 128-byte swizzle) brings [128 x 64] tiles of W and [Mpad x 64] tiles
//     of x into a ring of stages; an mbarrier per stage counts the bytes in.  The ring is as deep as the
//     shared memory of an SM allows for the CTAs that share it: 3 stages when three CTAs do, 9 for one alone.
//   * One thread issues four tcgen05.mma (K = 16 each) per stage and a tcgen05.commit that frees the
//     stage when they have read it.
//   * When N is small, a thread-block cluster of up to 8 CTAs splits K; the CTAs' partial sums are added
//     in rank order through distributed shared memory, so the result does not depend on timing.
//   * Epilogue: tcgen05.ld gives each thread the Mpad sums of its row of W; none / gated activation
//     (rows alternate 8 gate, 8 up: the partner sits 8 lanes away) / cap * tanh(v / cap); the sums are
//     turned through shared memory and leave as whole rows of out[M, N].
// Every wait is bounded: on a timeout the CTA records it (janis_tc05_timeouts), frees its tensor memory
// and returns.  No TMA load here uses cluster multicast.
#include <cooperative_groups.h>
#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace janis {
namespace tc {

constexpr int BLOCK_N = 128;          // rows of W per CTA (TMEM lanes)
constexpr int BLOCK_K = 64;           // bf16 elements per stage along K: one 128-byte swizzle row
constexpr int MIN_STAGES = 3;         // 73 KB a CTA: three CTAs share an SM, one's epilogue under the others' loads
constexpr int MAX_STAGES = 9;         // 217 KB: a CTA that has its SM to itself keeps nine tiles of W on the way
constexpr int MAX_M = 64;
constexpr int THREADS = 128;
constexpr int A_BYTES = BLOCK_N * BLOCK_K * 2;                    // 16 KB
constexpr int B_BYTES_MAX = MAX_M * BLOCK_K * 2;                  // 8 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES_MAX;
constexpr int smem_bytes(int stages) { return stages * STAGE_BYTES + 1024; }   // + room to align to 1024
static_assert(sizeof(float) * BLOCK_N * MAX_M <= MIN_STAGES * STAGE_BYTES, "the sums leave through the idle stages");

enum { EPI_NONE = 0, EPI_GATED_GELU = 1, EPI_SOFTCAP = 2, EPI_GATED_SILU = 3 };

__device__ int g_timeouts = 0;

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, int bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    // test_wait polls without suspending the thread (try_wait may park it for a while, which costs a stage's
    // worth of latency at every hand-over); about a second's worth of polls, then give up
    for (int it = 0; it < (1 << 26); ++it) {
        uint32_t done;
        asm volatile(
            "{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
// shared-memory operand: K-major rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);            // start address
    d |= (uint64_t)1 << 16;                             // leading byte offset (unused with a swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;                   // stride byte offset: next group of 8 rows
    d |= (uint64_t)1 << 46;                             // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                             // SWIZZLE_128B
    return d;
}
// kind::f16, bfloat16 operands both K-major, float accumulator, shape M x N x 16
__device__ __forceinline__ uint32_t instr_desc(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}

template <typename TO>
__global__ void __launch_bounds__(THREADS)
gemm_tc05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                 TO* __restrict__ out, int M, int Mpad, int N, int K, int split, int epi, float cap, int STAGES, int vec_ok) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * MAX_STAGES + 1];
    __shared__ uint32_t tmem_slot;
    __shared__ int failed;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = split > 1 ? (int)cg::this_cluster().block_rank() : 0;
    const int tile = blockIdx.x / split;
    const int n0 = tile * BLOCK_N;

    const uint32_t raw = (uint32_t)__cvta_generic_to_shared(smem_raw);
    const uint32_t stage0 = (raw + 1023) & ~1023u;                   // swizzle atoms want 1024-byte alignment
    unsigned char* stage_ptr = smem_raw + (stage0 - raw);
    const uint32_t bar_full = (uint32_t)__cvta_generic_to_shared(bars);
    const uint32_t bar_empty = bar_full + 8 * STAGES, bar_done = bar_full + 16 * STAGES;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(bar_full + 8 * i, 1); mbar_init(bar_empty + 8 * i, 1); }
        mbar_init(bar_done, 1);
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    const int tmem_cols = Mpad <= 32 ? 32 : 64;
    if (warp == 0) {                                                  // one warp allocates tensor memory
        const uint32_t slot = (uint32_t)__cvta_generic_to_shared(&tmem_slot);
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(slot), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = tmem_slot;

    // this CTA's share of K: tiles rank, rank + split, ...
    const int nk_all = (K + BLOCK_K - 1) / BLOCK_K;
    const int nk = rank < nk_all ? (nk_all - rank + split - 1) / split : 0;
    const int b_bytes = Mpad * BLOCK_K * 2;

    grid_dependents_launch();
    if (warp == 0 && lane == 0) {
        // ---- producer: TMA loads into the ring.  The weights are constants of the model: the first
        // tiles of W are on their way before this kernel waits for the one that produces x.
        const int pre = nk < STAGES ? nk : STAGES;
        for (int i = 0; i < pre; ++i) {
            mbar_expect_tx(bar_full + 8 * i, A_BYTES + b_bytes);
            tma_load_2d(stage0 + i * STAGE_BYTES, &map_w, (rank + i * split) * BLOCK_K, n0, bar_full + 8 * i);
        }
        grid_dependency_wait();
        for (int i = 0; i < pre; ++i)
            tma_load_2d(stage0 + i * STAGE_BYTES + A_BYTES, &map_x, (rank + i * split) * BLOCK_K, 0, bar_full + 8 * i);
        int s = pre == STAGES ? 0 : pre;                              // stage of tile i and how often it has been filled
        uint32_t fills = pre == STAGES ? 1 : 0;
        for (int i = pre; i < nk; ++i) {
            if (fills > 0 && !mbar_wait(bar_empty + 8 * s, (fills - 1) & 1)) { atomicExch(&failed, 1); break; }
            const uint32_t a = stage0 + s * STAGE_BYTES, b = a + A_BYTES;
            const int k0 = (rank + i * split) * BLOCK_K;
            mbar_expect_tx(bar_full + 8 * s, A_BYTES + b_bytes);
            tma_load_2d(a, &map_w, k0, n0, bar_full + 8 * s);
            tma_load_2d(b, &map_x, k0, 0, bar_full + 8 * s);
            if (++s == STAGES) { s = 0; ++fills; }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- the thread that issues the products
        grid_dependency_wait();
        const uint32_t idesc = instr_desc(BLOCK_N, Mpad);
        int s = 0;
        uint32_t round = 0;
        for (int i = 0; i < nk; ++i) {
            if (!mbar_wait(bar_full + 8 * s, round & 1)) { atomicExch(&failed, 1); break; }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const uint32_t a = stage0 + s * STAGE_BYTES, b = a + A_BYTES;
#pragma unroll
            for (int kk = 0; kk < BLOCK_K / 16; ++kk)                 // 32 bytes further along the swizzled row
                umma(tmem, smem_desc(a + kk * 32), smem_desc(b + kk * 32), idesc, (i > 0 || kk > 0) ? 1u : 0u);
            umma_commit(bar_empty + 8 * s);                           // the stage is free once these have read it
            if (++s == STAGES) { s = 0; ++round; }
        }
        umma_commit(bar_done);                                        // all products of this CTA have finished
    }
    else grid_dependency_wait();
    __syncwarp();
    // ---- everyone: wait for the accumulator
    bool ok = nk == 0 ? true : mbar_wait(bar_done, 0);
    ok = __syncthreads_and(ok ? 1 : 0) && failed == 0;
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");

    // the Mpad sums of row (32 * warp + lane) of this CTA's tile of W
    float acc[MAX_M];
#pragma unroll
    for (int i = 0; i < MAX_M; ++i) acc[i] = 0.f;
    if (ok && nk > 0) {
        const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16);
#pragma unroll
        for (int c = 0; c < MAX_M; c += 16) {
            if (c < Mpad) {
                uint32_t r[16];
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
                    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                      "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                    : "r"(taddr + c));
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[c + j] = __uint_as_float(r[j]);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(tmem_cols) : "memory");
    if (!ok && threadIdx.x == 0) atomicAdd(&g_timeouts, 1);

    // ---- K split over a cluster: partial sums through distributed shared memory, in rank order
    if (split > 1) {
        float* mine = reinterpret_cast<float*>(stage_ptr);            // [MAX_M][BLOCK_N]; the stages are idle now
#pragma unroll
        for (int m = 0; m < MAX_M; ++m)
            if (m < Mpad) mine[m * BLOCK_N + threadIdx.x] = acc[m];
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        if (rank == 0) {
            for (int r = 1; r < split; ++r) {
                const float* theirs = cluster.map_shared_rank(mine, r);
#pragma unroll
                for (int m = 0; m < MAX_M; ++m)
                    if (m < Mpad) acc[m] += theirs[m * BLOCK_N + threadIdx.x];
            }
        }
        cluster.sync();
        if (rank != 0) return;
    }
    if (!ok) return;

    // ---- epilogue: thread = row n of W holds out[0 .. M)[n].  Stored from here a warp would write 2 bytes to each
    // of 32 places per instruction (8.6 us a CTA, measured); the sums are turned through the idle stages instead
    // and leave as whole rows of the tile.
    float* turned = reinterpret_cast<float*>(stage_ptr);              // [M][cols]
    const bool gated = epi == EPI_GATED_GELU || epi == EPI_GATED_SILU;
    const int cols = gated ? BLOCK_N / 2 : BLOCK_N;                   // output columns of this tile
    const int n_cols = gated ? N / 2 : N, c0 = gated ? n0 / 2 : n0;   // columns of out, and the tile's first
    if (gated) {
        const bool gate_row = (threadIdx.x & 15) < 8;                 // rows alternate 8 gate, 8 up
        const int j = (threadIdx.x / 16) * 8 + (threadIdx.x & 7);
#pragma unroll
        for (int m = 0; m < MAX_M; ++m) {
            if (m < Mpad) {
                const float up = __shfl_down_sync(0xffffffffu, acc[m], 8);
                if (gate_row && m < M) {
                    const float g = acc[m];
                    const float act = epi == EPI_GATED_GELU ? gelu_tanh(g) : g / (1.0f + expf(-g));
                    turned[m * cols + j] = act * up;
                }
            }
        }
    } else {
#pragma unroll
        for (int m = 0; m < MAX_M; ++m) {
            if (m < M) {
                float v = acc[m];
                if (epi == EPI_SOFTCAP && cap > 0.f) v = cap * tanhf(v / cap);
                turned[m * cols + threadIdx.x] = v;
            }
        }
    }
    __syncthreads();
    constexpr int VEC = 16 / sizeof(TO);                              // values of a 16-byte store
    if (vec_ok) {
        const int per_row = cols / VEC;
        for (int idx = threadIdx.x; idx < M * per_row; idx += THREADS) {
            const int m = idx / per_row, c = (idx % per_row) * VEC;
            if (c0 + c >= n_cols) continue;                           // n_cols is a multiple of VEC here
            const float* src = turned + m * cols + c;
            TO* dst = out + (size_t)m * n_cols + c0 + c;
            if constexpr (sizeof(TO) == 2) {
                const float4 lo = *reinterpret_cast<const float4*>(src), hi = *reinterpret_cast<const float4*>(src + 4);
                __nv_bfloat162 p0 = __floats2bfloat162_rn(lo.x, lo.y), p1 = __floats2bfloat162_rn(lo.z, lo.w);
                __nv_bfloat162 p2 = __floats2bfloat162_rn(hi.x, hi.y), p3 = __floats2bfloat162_rn(hi.z, hi.w);
                uint4 w;
                w.x = *reinterpret_cast<uint32_t*>(&p0); w.y = *reinterpret_cast<uint32_t*>(&p1);
                w.z = *reinterpret_cast<uint32_t*>(&p2); w.w = *reinterpret_cast<uint32_t*>(&p3);
                *reinterpret_cast<uint4*>(dst) = w;
            } else {
                *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(src);
            }
        }
    } else {
        for (int idx = threadIdx.x; idx < M * cols; idx += THREADS) {
            const int m = idx / cols, c = idx % cols;
            if (c0 + c < n_cols) out[(size_t)m * n_cols + c0 + c] = from_float<TO>(turned[m * cols + c]);
        }
    }
}

// ---- host side: tensor maps
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiled encoder() {
    static EncodeTiled fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiled)p;
    });
    return fn;
}

// a [rows, K] bfloat16 matrix, K contiguous, in boxes of 64 x box_rows with the 128-byte swizzle
static bool make_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows) {
    EncodeTiled enc = encoder();
    if (!enc) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BLOCK_K, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static const CUtensorMap* cached_map(const void* ptr, int rows, int K, int box_rows) {
    static std::map<std::tuple<const void*, int, int, int>, CUtensorMap> cache;
    static std::mutex lock;
    std::lock_guard<std::mutex> guard(lock);
    auto key = std::make_tuple(ptr, rows, K, box_rows);
    auto it = cache.find(key);
    if (it == cache.end()) {
        CUtensorMap m;
        if (!make_map(&m, ptr, rows, K, box_rows)) return nullptr;
        it = cache.emplace(key, m).first;
    }
    return &it->second;
}

}  // namespace tc
}  // namespace janis

using namespace janis;

static int sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
    }
    return sms;
}

static int g_tc05_stages = 0;       // 0: chosen from the number of CTAs per SM

// Fixes the depth of the ring of stages (3 to 9; 0: automatic again).  For tests and tuning.
JANIS_EXPORT void janis_tc05_set_stages(int stages) {
    g_tc05_stages = stages <= 0 ? 0 : (stages < tc::MIN_STAGES ? tc::MIN_STAGES : (stages > tc::MAX_STAGES ? tc::MAX_STAGES : stages));
}

namespace janis { int gemv_push_timeouts_async(int* host, cudaStream_t stream); }      // gemv_bf16.cu

// The same count copied into `host` (pinned memory, two ints: this kernel's count, then that of the skinny products'
// clusters) in the order of `stream`, without waiting for it: a caller that waits for the stream anyway (for its
// tokens) finds the counts there afterwards.
JANIS_EXPORT int janis_tc05_timeouts_async(int* host, cudaStream_t stream) {
    cudaError_t e = cudaMemcpyFromSymbolAsync(host, tc::g_timeouts, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
    if (e != cudaSuccess) return fail("tc05_timeouts_async: %s", cudaGetErrorString(e));
    return janis::gemv_push_timeouts_async(host + 1, stream);
}

JANIS_EXPORT int janis_tc05_timeouts() {
    int n = -1;
    if (cudaMemcpyFromSymbol(&n, tc::g_timeouts, sizeof(int)) != cudaSuccess) return -1;
    return n;
}

// x [M, K] bf16 (16-byte aligned rows: K % 8 == 0), W [N, K] bf16, out [M, N] (or [M, N/2] with a gated epilogue),
// M <= 64.  split: CTAs of a cluster that share K (1, 2, 4, 8); 0 = chosen from N and K.
JANIS_EXPORT int janis_gemm_tc05(const void* x, const void* W, void* out, int out_dtype, int M, int N, int K, int epi,
                                 float cap, int split, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > tc::MAX_M) return fail("gemm_tc05: at most %d rows, found %d", tc::MAX_M, M);
    if (K <= 0 || K % 8) return fail("gemm_tc05: K must be a positive multiple of 8, found %d", K);
    if (out_dtype != JANIS_BF16 && out_dtype != JANIS_F32) return fail("gemm_tc05: unknown output dtype %d", out_dtype);
    if ((epi == tc::EPI_GATED_GELU || epi == tc::EPI_GATED_SILU) && N % 16)
        return fail("gemm_tc05: a gated epilogue needs N to be a multiple of 16, found %d", N);
    if (epi < 0 || epi > 3) return fail("gemm_tc05: unknown epilogue %d", epi);
    if (((uintptr_t)x | (uintptr_t)W) & 15) return fail("gemm_tc05: operands must be 16-byte aligned");
    if (split != 0 && split != 1 && split != 2 && split != 4 && split != 8)
        return fail("gemm_tc05: split must be 0, 1, 2, 4 or 8, found %d", split);
    const int Mpad = (M + 15) / 16 * 16;
    const int tiles = (N + tc::BLOCK_N - 1) / tc::BLOCK_N, nk = (K + tc::BLOCK_K - 1) / tc::BLOCK_K;
    if (split == 0) {
        // few tiles of W: K is shared by a cluster as long as each CTA keeps 16 tiles of it (measured in replayed
        // graphs: N = 4096 and 2304 with K = 2304 and 2048 are fastest with 2 CTAs, N = 2304 with K = 9216 with 4;
        // clusters of 8 were slower everywhere)
        split = 1;
        while (split < 4 && tiles * split * 2 <= sm_count() && nk >= split * 2 * 16) split *= 2;
    }
    const CUtensorMap* mw = tc::cached_map(W, N, K, tc::BLOCK_N);
    const CUtensorMap* mx = tc::cached_map(x, M, K, Mpad);
    if (!mw || !mx) return fail("gemm_tc05: cuTensorMapEncodeTiled is not available or refused the operands");
    static bool configured[2] = {false, false};
    const int oi = out_dtype == JANIS_BF16 ? 0 : 1;
    if (!configured[oi]) {
        const int most = tc::smem_bytes(tc::MAX_STAGES);
        cudaError_t e = oi == 0 ? cudaFuncSetAttribute(tc::gemm_tc05_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, most)
                                : cudaFuncSetAttribute(tc::gemm_tc05_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
        if (e != cudaSuccess) return fail("gemm_tc05: shared memory of %d bytes refused: %s", most, cudaGetErrorString(e));
        configured[oi] = true;
    }
    // The ring is as deep as the SM's shared memory allows for the CTAs that share it: three CTAs with 3 stages
    // each when there are that many, two with 4, or one with 9 (a CTA alone with 3 stages had one tile of W arrive
    // every 0.6 us: a third of the SM's share of the memory bandwidth).
    const int per_sm = (tiles * split + sm_count() - 1) / sm_count();
    int stages = per_sm >= 3 ? tc::MIN_STAGES : (per_sm == 2 ? 4 : tc::MAX_STAGES);
    if (split > 1 && stages > 4) stages = 4;    // clusters of CTAs with most of an SM's shared memory each are placed slowly
    if (g_tc05_stages > 0) stages = g_tc05_stages;
    const int n_cols = (epi == tc::EPI_GATED_GELU || epi == tc::EPI_GATED_SILU) ? N / 2 : N;
    const int vec = out_dtype == JANIS_BF16 ? 8 : 4;
    const int vec_ok = (n_cols % vec == 0 && ((uintptr_t)out & 15) == 0) ? 1 : 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles * split);
    cfg.blockDim = dim3(tc::THREADS);
    cfg.dynamicSmemBytes = tc::smem_bytes(stages);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = split;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (overlap_launches()) {            // the kernel may arrive while the one before it runs (see common.cuh)
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 2;
    }
    cudaError_t e;
    if (oi == 0)
        e = cudaLaunchKernelEx(&cfg, tc::gemm_tc05_kernel<bf16>, *mw, *mx, (bf16*)out, M, Mpad, N, K, split, epi, cap, stages, vec_ok);
    else
        e = cudaLaunchKernelEx(&cfg, tc::gemm_tc05_kernel<float>, *mw, *mx, (float*)out, M, Mpad, N, K, split, epi, cap, stages, vec_ok);
    if (e != cudaSuccess) return fail("gemm_tc05: launch failed: %s", cudaGetErrorString(e));
    return launched("gemm_tc05");
}
