// Skinny bfloat16 product for decoding: out[M, N] = x[M, K] * W[N, K]^T with M <= 64
// (one row per live sequence).  The step is bound by reading W once from HBM, so W
// is the 16-row operand of mma.sync.m16n8k16 and the batch rows are the 8-wide
// operand: every weight byte is read once, whatever M is.
//
// A tile of 16 rows of W belongs to one CTA, or to a thread-block cluster of CL CTAs
// when N is small (the o and down projections have few rows and long K): the warps of
// the cluster split K between them in blocks of 32, each CTA adds its warps' partial
// sums in warp order in its own shared memory, writes them into CTA 0's shared memory
// (distributed shared memory), and CTA 0 adds the CTAs' sums in rank order after one
// cluster barrier (tiles of more than 32 batch rows: CTA 0 reads them).  So more SMs pull on the same
// rows without any scratch in global memory, and a result does not depend on the grid
// beyond the fixed order of that sum.  Each thread reads 16 contiguous bytes of two
// rows of W straight into registers; the k order inside a block of 32 is permuted the
// same way for both operands, which leaves the dot product unchanged.
//
// Epilogues: none; gated activation over rows of W that alternate 8 gate rows and
// 8 up rows (one mma tile then holds matching pairs); cap * tanh(v / cap).
// Accumulation is float; the output is bfloat16 or float.  K must be a multiple of 8.
//
// The q/k/v projection of a decode step has a variant of its own (ROPE): a tile takes 8 rows of the first half
// of a head and the 8 rows half a head further on, so that one mma tile holds the pairs that the rotary encoding
// rotates; the epilogue rounds the sums to bfloat16 as the plain product would, rotates q and k by the angle of
// the token's position, writes q to its rows and k and v straight into the paged cache: the projection, the
// encoding and the cache write of a decode step are one kernel.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace janis {

#ifndef JANIS_GEMV_BULK_AHEAD
#define JANIS_GEMV_BULK_AHEAD 0       // 1: one bulk prefetch of the CTA's whole share of the tile instead (a tuning switch)
#endif
#ifndef JANIS_GEMV_AHEAD
#define JANIS_GEMV_AHEAD 1            // rounds of weights asked for before the wait (0: none; a tuning switch)
#endif

#ifndef JANIS_GEMV_PUSH
#define JANIS_GEMV_PUSH 2             // how a cluster adds up: 2 the other CTAs send their sums to CTA 0 with asynchronous stores that count on
                                      // its barrier, and leave; 1 they write them there and the cluster meets at one barrier; 0 CTA 0 reads them (two)
#endif
#ifndef JANIS_GEMV_U1
#define JANIS_GEMV_U1 4               // blocks of K a warp has in flight per round, up to 8 batch rows (a tuning switch)
#endif

constexpr int GEMV_WARPS = 8;        // warps of a CTA that split K (4 when N alone gives CTAs enough)

enum { EPI_NONE = 0, EPI_GATED_GELU = 1, EPI_SOFTCAP = 2, EPI_GATED_SILU = 3 };

// What the ROPE variant needs beside the product: the step's tables, the inverse frequencies and one cache line.
struct RopeStore {
    const int* tok_pos;        // [M] position of each row's token
    const int* tok_seq;        // [M] its sequence in the step
    const int* seq_slot;       // [n_seq] cache slot, < 0: padding (rotated, stored nowhere)
    const int* seq_end;        // [n_seq] tokens cached after the step
    const float* inv_freq;     // [hd / 2]
    bf16* kpool;               // [pages, nkv, PAGE, hd]; null: the rows hold queries alone
    bf16* vpool;
    const int* page_table;     // [slots, table_stride]
    int table_stride, ring_len, nq, nkv, hd;
    int row_heads;             // heads in a row of the output that takes the queries (nq, or nq + 2 nkv)
};

__device__ int g_push_timeouts = 0;     // how often CTA 0 of a cluster has given up the wait for the others' sums

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

template <int MT, int U, int CL, int NW, typename TO, bool ROPE = false>
__global__ void __launch_bounds__(NW * 32)
gemv_bf16_kernel(const bf16* __restrict__ x, const bf16* __restrict__ W, TO* __restrict__ out, int M, int N,
                 int K, int epi, float cap, const RopeStore rs) {
    __shared__ float red[NW][MT][32][4];
    __shared__ __align__(16) float cta_sum[MT * 128];        // this CTA's sum over its warps; read by CTA 0 of the cluster
    constexpr bool PUSH = JANIS_GEMV_PUSH && CL > 1 && MT <= 4;      // (the gather area of 8 row tiles does not fit)
    __shared__ __align__(16) float gather[PUSH ? CL : 1][PUSH ? MT * 128 : 1];     // in CTA 0 of a cluster: every CTA's sums, written by their owners
    constexpr bool ASYNC_PUSH = PUSH && JANIS_GEMV_PUSH == 2;
    __shared__ __align__(8) unsigned long long push_bar;          // in CTA 0: counts the bytes the other CTAs send
    if (ASYNC_PUSH) {
        if (threadIdx.x == 0 && cg::this_cluster().block_rank() == 0) {
            const uint32_t b = (uint32_t)__cvta_generic_to_shared(&push_bar);
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(b));
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(b), "r"((CL - 1) * MT * 128 * 4) : "memory");
            asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        }
        __syncthreads();
        asm volatile("barrier.cluster.arrive.aligned;\n" ::: "memory");           // "I am running", and CTA 0's barrier is set up
    } else if (PUSH) asm volatile("barrier.cluster.arrive.relaxed.aligned;\n" ::: "memory");   // "I am running": waited for before the push
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int rank = CL > 1 ? (int)cg::this_cluster().block_rank() : 0;
    const int tile = blockIdx.x / CL;
    const int r0 = tile * 16;
    // rows past the end read the last row; their results are never stored
    int row_lo = min(r0 + g, N - 1), row_hi = min(r0 + g + 8, N - 1);
    if (ROPE) {                                 // 8 rows of a head's first half and their partners half a head on
        const int tiles_per_head = rs.hd >> 4;
        row_lo = (tile / tiles_per_head) * rs.hd + (tile % tiles_per_head) * 8 + g;
        row_hi = row_lo + (rs.hd >> 1);
    }
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

    constexpr int SPLIT = NW * CL;             // warps that share the K of a tile
    const int nblk = (K + 31) / 32;
    // Weights are constants of the model: the first round of them is asked for (into L2) before
    // this kernel waits for the one that produces x.
    uint4 a_lo[U], a_hi[U];
    auto load_w = [&](int kb0) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k0 = (kb0 + u * SPLIT) * 32;
            const bool in = k0 + t * 8 < K;          // K % 8 == 0: a 16-byte piece is all in or all out
            a_lo[u] = in ? ldg_stream(wlo + k0) : make_uint4(0, 0, 0, 0);
            a_hi[u] = in ? ldg_stream(whi + k0) : make_uint4(0, 0, 0, 0);
        }
    };
    int kb = rank * NW + warp;
    grid_dependents_launch();
    // ROPE: thread idx of the CTA that ends up with the sums has the pair (i, ln, p) of the epilogue below; its
    // angle comes from the step's tables and the model's constants, so it is computed before the wait
    float rope_sin = 0.f, rope_cos = 1.f;
    if (ROPE && rank == 0 && threadIdx.x < MT * 64) {
        const int i = threadIdx.x / 64, ln = (threadIdx.x / 2) % 32, p = threadIdx.x % 2;
        const int m = i * 8 + (ln & 3) * 2 + p;
        const int tiles_per_head = rs.hd >> 4;
        const int head = tile / tiles_per_head, d = (tile % tiles_per_head) * 8 + (ln >> 2);
        if (m < M && head < rs.nq + rs.nkv) sincosf((float)rs.tok_pos[m] * rs.inv_freq[d], &rope_sin, &rope_cos);
    }
#if JANIS_GEMV_BULK_AHEAD
    // The 16 rows of a tile lie one after another in memory: one bulk prefetch per CTA asks for this CTA's
    // share of them (into L2) while the kernel before this one still runs.
    if (threadIdx.x == 0) {
        const int rows_here = min(16, N - r0);
        const size_t bytes = (size_t)rows_here * K * sizeof(bf16);
        size_t piece = ((bytes / CL) + 15) & ~(size_t)15;
        const size_t off = piece * rank;
        if (off < bytes) {
            if (off + piece > bytes) piece = (bytes - off) & ~(size_t)15;
            if (piece > 0)
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(reinterpret_cast<const char*>(W + (size_t)r0 * K) + off),
                             "r"((uint32_t)piece) : "memory");
        }
    }
#elif JANIS_GEMV_AHEAD
    // hints only: a load into registers would have to land before the wait below lets the thread go on
    for (int pk = kb, n = 0; pk < nblk && n < JANIS_GEMV_AHEAD * U; pk += SPLIT, ++n) {
        const int k0 = pk * 32;
        if (k0 + t * 8 < K) {
            asm volatile("prefetch.global.L2 [%0];\n" ::"l"(wlo + k0));
            asm volatile("prefetch.global.L2 [%0];\n" ::"l"(whi + k0));
        }
    }
#endif
    grid_dependency_wait();
    for (; kb < nblk; kb += SPLIT * U) {
        uint4 b[U][MT];
        load_w(kb);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k0 = (kb + u * SPLIT) * 32;
            const bool in = k0 + t * 8 < K;
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
    // the CTA's sum, warps in index order; layout [tile i][lane][c]
    for (int idx = threadIdx.x; idx < MT * 128; idx += blockDim.x) {
        const int i = idx / 128, ln = (idx / 4) % 32, c = idx % 4;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) v += red[w][i][ln][c];
        cta_sum[idx] = v;
    }
    if (ASYNC_PUSH) {
        // The other CTAs send their sums to CTA 0's shared memory with asynchronous stores that count their bytes on
        // CTA 0's barrier, and are done; CTA 0 waits for the bytes alone (no barrier of the whole cluster; the wait is
        // bounded) and adds the sums in rank order.  Against one barrier of the cluster: 2.423 -> 2.407 ms a decode
        // step at batch 8, 1.686 -> 1.655 ms at batch 1 (78 such products a step).
        asm volatile("barrier.cluster.wait.aligned;\n" ::: "memory");
        __syncthreads();
        if (rank != 0) {
            uint32_t dst, bar;
            const uint32_t ldst = (uint32_t)__cvta_generic_to_shared(&gather[rank][0]);
            const uint32_t lbar = (uint32_t)__cvta_generic_to_shared(&push_bar);
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(dst) : "r"(ldst), "r"(0));
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(bar) : "r"(lbar), "r"(0));
            for (int idx = threadIdx.x; idx < MT * 32; idx += blockDim.x) {
                const float4 v = *reinterpret_cast<const float4*>(&cta_sum[idx * 4]);
                asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];\n" ::"r"(
                                 dst + idx * 16),
                             "r"(__float_as_uint(v.x)), "r"(__float_as_uint(v.y)), "r"(__float_as_uint(v.z)), "r"(__float_as_uint(v.w)),
                             "r"(bar)
                             : "memory");
            }
            return;
        }
        if (threadIdx.x == 0) {
            const uint32_t b = (uint32_t)__cvta_generic_to_shared(&push_bar);
            uint32_t done = 0;
            for (int tries = 0; tries < (1 << 22) && !done; ++tries)
                asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], 0;\nselp.u32 %0, 1, 0, p;\n}\n"
                             : "=r"(done) : "r"(b) : "memory");
            if (!done) atomicAdd(&g_push_timeouts, 1);
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < MT * 128; idx += blockDim.x) {
            float v = cta_sum[idx];
#pragma unroll
            for (int r = 1; r < CL; ++r) v += gather[r][idx];   // rank order
            red[0][idx / 128][(idx / 4) % 32][idx % 4] = v;
        }
    } else if (PUSH) {
        // every CTA writes its sums into CTA 0's shared memory (all CTAs of the cluster are running: the
        // barrier they arrived at when they started), one cluster barrier publishes them, CTA 0 adds them
        // in rank order and the others are done
        cg::cluster_group cluster = cg::this_cluster();
        asm volatile("barrier.cluster.wait.aligned;\n" ::: "memory");
        float* dst = cluster.map_shared_rank(&gather[0][0], 0) + rank * MT * 128;
        __syncthreads();
        for (int idx = threadIdx.x; idx < MT * 128; idx += blockDim.x) dst[idx] = cta_sum[idx];
        cluster.sync();
        if (rank != 0) return;
        for (int idx = threadIdx.x; idx < MT * 128; idx += blockDim.x) {
            float v = gather[0][idx];
#pragma unroll
            for (int r = 1; r < CL; ++r) v += gather[r][idx];   // rank order
            red[0][idx / 128][(idx / 4) % 32][idx % 4] = v;
        }
    } else if (CL > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();                              // every CTA's sum is in its shared memory
        if (rank == 0) {
            for (int idx = threadIdx.x; idx < MT * 128; idx += blockDim.x) {
                float v = cta_sum[idx];
#pragma unroll
                for (int r = 1; r < CL; ++r) v += cluster.map_shared_rank(cta_sum, r)[idx];   // rank order
                red[0][idx / 128][(idx / 4) % 32][idx % 4] = v;
            }
        }
        cluster.sync();                              // nobody leaves while its shared memory is being read
        if (rank != 0) return;
    } else {
        __syncthreads();
        for (int idx = threadIdx.x; idx < MT * 128; idx += blockDim.x)
            red[0][idx / 128][(idx / 4) % 32][idx % 4] = cta_sum[idx];
    }
    __syncthreads();
    const float (*tot)[32][4] = red[0];             // the tile's full sums

    if (ROPE) {
        // rows g of the tile are elements d of a head, rows g + 8 elements d + hd/2: a rotary pair per (token, g)
        static_assert(!ROPE || MT * 64 <= NW * 32, "one pair per thread");
        if (threadIdx.x < MT * 64) {
            const int i = threadIdx.x / 64, ln = (threadIdx.x / 2) % 32, p = threadIdx.x % 2;
            const int m = i * 8 + (ln & 3) * 2 + p;
            if (m < M) {
                const int hd = rs.hd, half = hd >> 1, tiles_per_head = hd >> 4;
                const int head = tile / tiles_per_head, d = (tile % tiles_per_head) * 8 + (ln >> 2);
                // rounded to bfloat16 first, as the plain product followed by the encoding kernel rounds them
                float lo = __bfloat162float(__float2bfloat16(tot[i][ln][p]));
                float hi = __bfloat162float(__float2bfloat16(tot[i][ln][p + 2]));
                const bool is_v = head >= rs.nq + rs.nkv;
                if (!is_v) {
                    rotate_pair(lo, hi, rope_sin, rope_cos, lo, hi);
                }
                if (head < rs.nq) {
                    bf16* q = reinterpret_cast<bf16*>(out) + ((size_t)m * rs.row_heads + head) * hd + d;
                    q[0] = __float2bfloat16(lo);
                    q[half] = __float2bfloat16(hi);
                } else {
                    const int seq = rs.tok_seq[m];
                    const int slot = rs.seq_slot[seq];
                    const int pos = rs.tok_pos[m];
                    int idx = pos;
                    bool keep = slot >= 0;
                    if (keep && rs.ring_len > 0) {
                        keep = pos >= rs.seq_end[seq] - rs.ring_len;
                        idx = pos % rs.ring_len;
                    }
                    if (keep) {
                        const int kvh = is_v ? head - rs.nq - rs.nkv : head - rs.nq;
                        const int page = rs.page_table[(size_t)slot * rs.table_stride + idx / JANIS_PAGE];
                        bf16* dst = (is_v ? rs.vpool : rs.kpool) +
                                    (((size_t)page * rs.nkv + kvh) * JANIS_PAGE + idx % JANIS_PAGE) * hd + d;
                        dst[0] = __float2bfloat16(lo);
                        dst[half] = __float2bfloat16(hi);
                    }
                }
            }
        }
        return;
    }

    if (epi == EPI_GATED_GELU || epi == EPI_GATED_SILU) {
        // rows g of the tile are gate rows, rows g + 8 the matching up rows
        const int I = N / 2;
        for (int idx = threadIdx.x; idx < MT * 32 * 2; idx += blockDim.x) {
            const int i = idx / 64, ln = (idx / 2) % 32, p = idx % 2;
            const float gate = tot[i][ln][p], up = tot[i][ln][p + 2];
            const int m = i * 8 + (ln & 3) * 2 + p;
            const int j = tile * 8 + (ln >> 2);
            if (m < M && j < I) {
                const float a = epi == EPI_GATED_GELU ? gelu_tanh(gate) : gate / (1.0f + expf(-gate));
                out[(size_t)m * I + j] = from_float<TO>(a * up);
            }
        }
        return;
    }
    for (int idx = threadIdx.x; idx < MT * 32 * 4; idx += blockDim.x) {
        const int i = idx / 128, ln = (idx / 4) % 32, c = idx % 4;
        float v = tot[i][ln][c];
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

static int g_gemv_small_ctas = 1;
// tuning switch: 0 launches tall products with 8-warp CTAs too
JANIS_EXPORT void janis_gemv_small_ctas(int on) { g_gemv_small_ctas = on ? 1 : 0; }

template <int MT, int U, int CL, typename TO, bool ROPE = false>
static int launch_one(const bf16* x, const bf16* W, TO* out, int M, int N, int K, int epi, float cap,
                      const RopeStore& rs, cudaStream_t stream) {
    const int tiles = (N + 15) / 16;
    if (CL == 1) {
        // many tiles: CTAs of 4 warps, so that more of them are resident and the last wave is short
        if (tiles >= 1024 && g_gemv_small_ctas && !ROPE)
            return launch_kernel("gemv_bf16", gemv_bf16_kernel<MT, U, 1, 4, TO, false>, dim3(tiles), dim3(4 * 32), 0, stream, 1,
                                 x, W, out, M, N, K, epi, cap, rs);
        return launch_kernel("gemv_bf16", gemv_bf16_kernel<MT, U, 1, GEMV_WARPS, TO, ROPE>, dim3(tiles), dim3(GEMV_WARPS * 32), 0,
                             stream, 1, x, W, out, M, N, K, epi, cap, rs);
    }
    return launch_kernel("gemv_bf16", gemv_bf16_kernel<MT, U, CL, GEMV_WARPS, TO, ROPE>, dim3(tiles * CL), dim3(GEMV_WARPS * 32),
                         0, stream, CL, x, W, out, M, N, K, epi, cap, rs);
}

template <int MT, int U>
static int launch_gemv(const bf16* x, const bf16* W, void* out, int out_dtype, int M, int N, int K, int epi,
                       float cap, int cluster, cudaStream_t stream) {
    const RopeStore none = {};
#define JANIS_GEMV(CL)                                                                                                \
    (out_dtype == JANIS_BF16 ? launch_one<MT, U, CL, bf16>(x, W, (bf16*)out, M, N, K, epi, cap, none, stream)          \
                             : launch_one<MT, U, CL, float>(x, W, (float*)out, M, N, K, epi, cap, none, stream))
    if (cluster >= 4) return JANIS_GEMV(4);
    if (cluster >= 2) return JANIS_GEMV(2);
    return JANIS_GEMV(1);
#undef JANIS_GEMV
}

template <int MT, int U>
static int launch_gemv_rope(const bf16* x, const bf16* W, bf16* out, int M, int N, int K, int cluster,
                            const RopeStore& rs, cudaStream_t stream) {
    if (cluster >= 4) return launch_one<MT, U, 4, bf16, true>(x, W, out, M, N, K, EPI_NONE, 0.f, rs, stream);
    if (cluster >= 2) return launch_one<MT, U, 2, bf16, true>(x, W, out, M, N, K, EPI_NONE, 0.f, rs, stream);
    return launch_one<MT, U, 1, bf16, true>(x, W, out, M, N, K, EPI_NONE, 0.f, rs, stream);
}

static int choose_cluster(int tiles, int nblk) {
    // enough CTAs to fill the GPU a few times over, as long as every warp keeps some blocks of K.  Measured in a
    // replayed graph at 2304 x 2048 / 4096 x 2304 / 2304 x 9216: clusters of 4 / 2 / 4 are fastest (5.1, 7.5, 11.5 us;
    // the qkv product takes 9.2 us with 4, every one is slower with 8).
    int cluster = 1;
    while (cluster < 4 && tiles * cluster < 512 && nblk >= GEMV_WARPS * cluster * 2 * 2) cluster *= 2;
    return cluster;
}

// x [M, K] bf16, W [N, K] bf16, out [M, N] (or [M, N/2] with a gated epilogue).
// cluster: CTAs that share a tile's K (1, 2 or 4); 0 lets the kernel choose from N and K.
JANIS_EXPORT int janis_gemv_bf16(const void* x, const void* W, void* out, int out_dtype, int M, int N, int K,
                                 int epi, float cap, int cluster, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64) return fail("gemv_bf16: at most 64 rows, found %d", M);
    if (K <= 0 || K % 8) return fail("gemv_bf16: K must be a positive multiple of 8, found %d", K);
    if (out_dtype != JANIS_BF16 && out_dtype != JANIS_F32) return fail("gemv_bf16: unknown output dtype %d", out_dtype);
    if ((epi == EPI_GATED_GELU || epi == EPI_GATED_SILU) && N % 16)
        return fail("gemv_bf16: a gated epilogue needs N to be a multiple of 16, found %d", N);
    if (epi < 0 || epi > 3) return fail("gemv_bf16: unknown epilogue %d", epi);
    if (cluster != 0 && cluster != 1 && cluster != 2 && cluster != 4)
        return fail("gemv_bf16: cluster must be 0, 1, 2 or 4, found %d", cluster);
    if (((uintptr_t)x | (uintptr_t)W) & 15) return fail("gemv_bf16: operands must be 16-byte aligned");
    const bf16* xp = (const bf16*)x;
    const bf16* wp = (const bf16*)W;
    const int tiles = (N + 15) / 16, nblk = (K + 31) / 32;
    if (cluster == 0) cluster = choose_cluster(tiles, nblk);
    if (M <= 8) return launch_gemv<1, JANIS_GEMV_U1>(xp, wp, out, out_dtype, M, N, K, epi, cap, cluster, stream);
    if (M <= 16) return launch_gemv<2, 4>(xp, wp, out, out_dtype, M, N, K, epi, cap, cluster, stream);
    if (M <= 32) return launch_gemv<4, 2>(xp, wp, out, out_dtype, M, N, K, epi, cap, cluster, stream);
    return launch_gemv<8, 1>(xp, wp, out, out_dtype, M, N, K, epi, cap, cluster, stream);
}

// The q/k/v projection of a decode step with the rotary encoding and the cache write in its epilogue (bfloat16,
// at most 16 rows, the whole head rotated: rot == hd, hd a multiple of 16).  x [M, K]; W [heads * hd, K] with
// heads = nq + 2 nkv (kpool given) or nq (kpool null: a layer that reads another layer's keys); q goes to
// q_out [M, row_heads, hd], k and v to the cache line as janis_rope_store writes them.
JANIS_EXPORT int janis_gemv_rope_store(const void* x, const void* W, void* q_out, int M, int K, const int* tok_pos,
                                       const int* tok_seq, const int* seq_slot, const int* seq_end,
                                       const float* inv_freq, int nq, int nkv, int hd, int row_heads, void* kpool,
                                       void* vpool, const int* page_table, int table_stride, int ring_len,
                                       cudaStream_t stream) {
    if (M <= 0) return 0;
    if (M > 16) return fail("gemv_rope_store: at most 16 rows, found %d", M);
    if (K <= 0 || K % 8) return fail("gemv_rope_store: K must be a positive multiple of 8, found %d", K);
    if (hd <= 0 || hd % 16) return fail("gemv_rope_store: the head size must be a multiple of 16, found %d", hd);
    if (nq <= 0 || nkv < 0 || row_heads < nq) return fail("gemv_rope_store: %d query heads in rows of %d heads", nq, row_heads);
    if (((uintptr_t)x | (uintptr_t)W) & 15) return fail("gemv_rope_store: operands must be 16-byte aligned");
    const int heads = kpool != nullptr ? nq + 2 * nkv : nq;
    const int N = heads * hd;
    RopeStore rs = {};
    rs.tok_pos = tok_pos; rs.tok_seq = tok_seq; rs.seq_slot = seq_slot; rs.seq_end = seq_end; rs.inv_freq = inv_freq;
    rs.kpool = (bf16*)kpool; rs.vpool = (bf16*)vpool; rs.page_table = page_table;
    rs.table_stride = table_stride; rs.ring_len = ring_len;
    rs.nq = nq; rs.nkv = kpool != nullptr ? nkv : 0; rs.hd = hd; rs.row_heads = row_heads;
    const int cluster = choose_cluster(N / 16, (K + 31) / 32);
    if (M <= 8)
        return launch_gemv_rope<1, JANIS_GEMV_U1>((const bf16*)x, (const bf16*)W, (bf16*)q_out, M, N, K, cluster, rs, stream);
    return launch_gemv_rope<2, 4>((const bf16*)x, (const bf16*)W, (bf16*)q_out, M, N, K, cluster, rs, stream);
}

// How often CTA 0 of a cluster has given up the wait for the other CTAs' sums, copied into `host` in the order of
// `stream` without waiting for it.
namespace janis {
int gemv_push_timeouts_async(int* host, cudaStream_t stream) {
    cudaError_t e = cudaMemcpyFromSymbolAsync(host, g_push_timeouts, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
    return e == cudaSuccess ? 0 : fail("gemv_push_timeouts_async: %s", cudaGetErrorString(e));
}
}  // namespace janis
