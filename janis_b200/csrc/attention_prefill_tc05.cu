// Prompt attention in bfloat16 on the 5th-generation tensor cores, for head sizes that are a multiple
// of 64 up to 256; one head size per compiled library (JANIS_HEAD_DIM).
//
// A CTA owns 128 queries of one sequence and one query head and walks the tiles of 64 keys that the
// causal mask and the window leave (the tiling, the sharing of long tiles between CTAs and the merge
// are those of attention_prefill_mma.cu).  Three roles:
//   * one thread brings Q once and then K and V tiles by TMA tensor maps (128-byte swizzle, slabs of 64
//     features) into rings of two stages each;
//   * two threads issue tcgen05.mma, each on its own: one S = Q K^T (K-major operands from shared memory) into
//     one of two [128 x 64] float buffers in tensor memory, the other O += P V (P from tensor memory, V from
//     shared memory as the MN-major operand: its rows are keys) into a [128 x head size] float accumulator
//     in tensor memory.  Issuing a product costs a thread 85 to 110 cycles (a tile has twenty of them): one
//     thread for both spent 1,900 of a tile's 3,400 cycles issuing;
//   * sixteen warps do the softmax, four threads per query row (tensor-memory lane = row; a thread takes
//     16 of a tile's 64 keys): tcgen05.ld of the scores, scale, cap * tanh, masks on absolute positions,
//     the row's maximum through shared memory, exponentials, P rounded to bfloat16 into one of two
//     buffers in tensor memory (pairs of keys per 32-bit column) for the second product.  With one buffer of
//     P (in shared memory) the softmax of a tile had to wait for the products of the tile before.  Four
//     softmax warps per scheduler hide each other's latencies; with one the kernel ran at a sixth of an
//     instruction per cycle.
// The scores run two tiles ahead of P V, and every softmax thread has two tiles in flight: it takes tile
// i + 1 out of tensor memory, caps and masks it and publishes its maximum before it turns tile i into P, so
// that it waits neither for the products nor for the other threads of its row.  The accumulator is
// rescaled only when a row's maximum has grown by more than 2^8 since the reference the exponentials
// use (P stays below 256, far inside bfloat16 and float range), so most tiles leave it untouched.
// Barriers and tensor memory are set up, and the CTA's place in the step is read from the step's tables, before
// the kernel waits for the one ahead of it in the stream; Q and the first keys are asked for right after the wait.
// A sequence's result depends on its own rows alone: keys beyond its end are masked by selection, and the rows of
// the last box of values that lie beyond its end are cleared in shared memory before P V reads them.
// Every wait is bounded: on a timeout the CTA records it (janis_attn_tc05_timeouts), frees its tensor
// memory and returns.  No TMA load here uses cluster multicast.
#include <cuda.h>

#include <algorithm>
#include <map>
#include <mutex>
#include <tuple>

#include "attention_prefill_tiles.cuh"

namespace janis {
namespace pt {

using pf::BM;
using pf::BN;
using pf::HD;

constexpr bool SUPPORTED = pf::TC05_HEAD;
constexpr int SLABS = SUPPORTED ? HD / 64 : 1;        // slabs of 64 features: one 128-byte swizzle row each
constexpr int Q_SLAB = BM * 128;                      // bytes
constexpr int KV_SLAB = BN * 128;
constexpr int Q_BYTES = SLABS * Q_SLAB;
constexpr int KV_TILE = SLABS * KV_SLAB;              // one of K or V, one stage
constexpr int STAGES = 2;
constexpr int SMEM_BYTES = 1024 + Q_BYTES + STAGES * 2 * KV_TILE;
constexpr int TMEM_COLS = HD + 192 <= 256 ? 256 : 512;        // O, two buffers of S, two of P (bfloat16 pairs: 32 columns each)
#ifndef JANIS_PT_SPLIT
#define JANIS_PT_SPLIT 4
#endif
constexpr int SPLIT = JANIS_PT_SPLIT;                 // threads that share a query row in the softmax (each 64 / SPLIT keys)
constexpr int CPT = 64 / SPLIT;                       // keys per softmax thread and tile: 16
static_assert(SPLIT == 4, "the softmax works in pieces of 16 columns");
constexpr int SOFTMAX_WARPS = 4 * SPLIT;              // warp w: rows 32 (w % 4) .., keys CPT (w / 4) .. of a tile
constexpr int LOADER_WARP = SOFTMAX_WARPS, ISSUER_WARP = SOFTMAX_WARPS + 1, PV_WARP = SOFTMAX_WARPS + 2;
constexpr int THREADS = (SOFTMAX_WARPS + 3) * 32;
constexpr int OCOLS = HD / SPLIT;                     // accumulator columns a softmax thread looks after
constexpr float RESCALE_STEP = 8.0f;                  // in units of log2: P stays below 2^8
// The softmax's work per score is what bounds this kernel, most of it on the special-function unit (16 results a
// cycle and SM, against 128 fused multiply-adds).  Two switches take work off it:
//   JANIS_PT_TANH_APPROX: the cap's tanh as one tanh.approx (relative error 2^-11, on scores that the product with V
//     weighs by P rounded to bfloat16, relative error 2^-9) instead of 2^x and 1/x;
//   JANIS_PT_POLY_EX2: every second exponential of the softmax as a cubic on the fused multiply-add pipe (relative
//     error 9e-5: the integer part goes into the exponent field, the fraction through the polynomial).
// Measured on a B200 at head size 256 (4 x 4,096 tokens, one launch): both off 425 us, tanh.approx alone 372 us,
// the cubic alone 444 us: the softmax warps are short of issue slots as much as of special-function results, and
// the cubic costs seven instructions for the one it saves.  So the first is on and the second stays a switch.
#ifndef JANIS_PT_TANH_APPROX
#define JANIS_PT_TANH_APPROX 1
#endif
#ifndef JANIS_PT_POLY_EX2
#define JANIS_PT_POLY_EX2 0
#endif

__device__ __forceinline__ float tanh_approx(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
// 2^x for x <= 8 without the special-function unit; 2^x = 0 below -126 (masked scores are -inf)
__device__ __forceinline__ float ex2_poly(float x) {
    const float MAGIC = 12582912.0f;                  // 1.5 x 2^23: adding it leaves the nearest integer in the low bits
    const float xc = fmaxf(x, -127.0f);
    const float t = (xc - 0.5f) + MAGIC;              // nearest integer to x - 0.5: floor(x), or x itself at a tie
    const float f = xc - (t - MAGIC);                 // in [0, 1]
    const float p = fmaf(fmaf(fmaf(0.077119089663028717f, f, 0.227564394474029541f), f, 0.695146143436431885f), f, 1.0f);
    const float r = __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
    return x < -126.0f ? 0.f : r;
}

enum { Q_FULL = 0, K_FULL = 1, K_EMPTY = 3, V_FULL = 5, V_EMPTY = 7, S_FULL = 9, S_EMPTY = 11, P_FULL = 13, O_DONE = 15, ROW_X = 17, N_BARS = 19 };

__device__ int g_timeouts = 0;

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, int bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
// try_wait parks the thread until the phase completes or the hinted time has passed (without the hint it came
// back after about a hundred cycles, and nineteen warps polling took issue slots from the ones that compute);
// a bounded number of tries, then give up.  `failed` lets the other roles give up sooner.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const volatile int* failed) {
    for (int it = 0; it < (1 << 18); ++it) {
        uint32_t done;
        asm volatile(
            "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done)
            : "r"(bar), "r"(parity), "r"(2000u)        // nanoseconds
            : "memory");
        if (done) return true;
        if ((it & 15) == 15 && *failed) return false;
    }
    return false;
}
// one arrival per warp: the lanes' writes are ordered before it by the warp barrier
__device__ __forceinline__ void warp_arrive(uint32_t bar, int lane) {
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
// Shared-memory operand in rows of 128 bytes with the 128-byte swizzle, groups of 8 rows 1024 bytes apart
// (the stride byte offset).  K-major operands (Q, K, P) walk along a row and never leave their slab within
// an instruction; the MN-major operand (V) has its K index on the rows and its N index runs on into the next
// slabs of 64 features, `lbo` bytes apart (the leading byte offset).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo = 1024) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);            // start address
    d |= (uint64_t)(lbo >> 4) << 16;                    // leading byte offset
    d |= (uint64_t)(1024 >> 4) << 32;                   // stride byte offset
    d |= (uint64_t)1 << 46;                             // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                             // SWIZZLE_128B
    return d;
}
// kind::f16, bfloat16 operands, float accumulator, shape M x N x 16; b_mn: the second operand is MN-major
__device__ __forceinline__ uint32_t instr_desc(int M, int N, bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// the same with the first operand in tensor memory (row i in lane i, two bfloat16 of K per 32-bit column)
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(tmem_d),
        "r"(tmem_a), "l"(b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
        "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
        "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
        "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};\n" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
                 "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

template <bool CAPPED>                                // CAPPED: scores go through cap * tanh(s / cap)
__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tc05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                         const int* __restrict__ seq_first_row, const int* __restrict__ seq_len, int n_seq,
                         bf16* __restrict__ out, int nq, int nkv, int kv_k_head0, float scale, float cap, int window,
                         int parts, int piece, float* __restrict__ partial) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[N_BARS];
    __shared__ uint32_t tmem_slot;
    __shared__ int failed;
    // the threads of a row tell each other their maxima; four tiles' worth, since a warp writes tile i + 1 while
    // another may still read tile i - 1 (it cannot be behind by more: tile i - 1's exchange needs its arrival)
    __shared__ float row_max[4][SPLIT][BM];
    __shared__ float row_sum[SPLIT][BM];             // and, at the end, their sums
    // Which sequence, which tile of queries, which part of its keys (as in the mma.sync kernel).  The step's
    // tables were written before the kernel ahead of this one started, so all of the set-up below (barriers,
    // tensor memory) runs while that kernel still does; the wait comes before the first load of Q.
    const int item = (int)gridDim.y - 1 - (int)blockIdx.y;
    const int gtile = item / parts, part = item % parts;
    int seq = -1, q0 = 0, len = 0;
    if (!pf::find_tile(gtile, seq_len, n_seq, seq, q0, len)) return;
    const int head = blockIdx.x;
    const int kvh = head / (nq / nkv);
    const int first = seq_first_row[seq];
    int k_first, n_tiles;
    pf::key_tiles(q0, len, window, k_first, n_tiles);
    const int np = pf::parts_of(n_tiles, parts, piece);
    const bool shared_tile = np > 1;
    if (part >= np) return;
    if (shared_tile) {
        const int t0 = (int)((long long)n_tiles * part / np), t1 = (int)((long long)n_tiles * (part + 1) / np);
        k_first += t0 * BN;
        n_tiles = t1 - t0;
    }

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t raw = (uint32_t)__cvta_generic_to_shared(smem_raw);
    const uint32_t sQ = (raw + 1023) & ~1023u;        // swizzle atoms want 1024-byte alignment
    const uint32_t sKV = sQ + Q_BYTES;                // stage s: K at sKV + s * 2 KV_TILE, V right after
    const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(bars);
    auto bar = [&](int i) { return bar0 + 8 * i; };

    if (warp == LOADER_WARP && lane == 0) {           // the loader sets the barriers up: it is their first user
        mbar_init(bar(Q_FULL), 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar(K_FULL + i), 1);
            mbar_init(bar(K_EMPTY + i), 1);
            mbar_init(bar(V_FULL + i), 1);
            mbar_init(bar(V_EMPTY + i), 1);
            mbar_init(bar(S_FULL + i), 1);
            mbar_init(bar(S_EMPTY + i), SOFTMAX_WARPS);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar(P_FULL + i), SOFTMAX_WARPS);
            mbar_init(bar(O_DONE + i), 1);
        }
        mbar_init(bar(ROW_X), SOFTMAX_WARPS);
        mbar_init(bar(ROW_X + 1), SOFTMAX_WARPS);
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == ISSUER_WARP) {                        // one warp allocates tensor memory
        const uint32_t slot = (uint32_t)__cvta_generic_to_shared(&tmem_slot);
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(slot), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    grid_dependents_launch();
    grid_dependency_wait();
    if (warp == LOADER_WARP && lane == 0) {           // Q and the first keys are on their way before the others are ready
        mbar_expect_tx(bar(Q_FULL), Q_BYTES);
        for (int sl = 0; sl < SLABS; ++sl) tma_load_2d(sQ + sl * Q_SLAB, &map_q, head * HD + sl * 64, first + q0, bar(Q_FULL));
        for (int i = 0; i < 2 && i < n_tiles; ++i) {
            mbar_expect_tx(bar(K_FULL + i), KV_TILE);
            for (int sl = 0; sl < SLABS; ++sl)
                tma_load_2d(sKV + i * 2 * KV_TILE + sl * KV_SLAB, &map_kv, (kv_k_head0 + kvh) * HD + sl * 64,
                            first + k_first + i * BN, bar(K_FULL + i));
        }
    }
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = tmem_slot;
    const uint32_t tO = tmem, tS = tmem + HD, tP = tS + 128;   // S buffer b at tS + 64 b, P buffer b at tP + 32 b
    const volatile int* fail_flag = &failed;

    if (warp == LOADER_WARP && lane == 0) {
        // ---- loader.  A tile of keys is free again as soon as its scores are done, and those run two tiles ahead
        // of P V, which frees the values: the loads follow the order in which the products finish
        // (K0 K1 V0 V1 K2 K3, then V(i + 2) after O(i) and K(i + 4) after S(i + 2), which is done by then), so
        // that a wait for values never holds back the keys that the next scores want.
        bool ok = true;
        auto load_k = [&](int i) {
            if (!ok || i >= n_tiles) return;
            const int s = i & 1;
            if (i >= 2 && !mbar_wait(bar(K_EMPTY + s), ((i >> 1) - 1) & 1, fail_flag)) { ok = false; return; }
            const uint32_t sK = sKV + s * 2 * KV_TILE;
            mbar_expect_tx(bar(K_FULL + s), KV_TILE);
            for (int sl = 0; sl < SLABS; ++sl)
                tma_load_2d(sK + sl * KV_SLAB, &map_kv, (kv_k_head0 + kvh) * HD + sl * 64, first + k_first + i * BN, bar(K_FULL + s));
        };
        auto load_v = [&](int i) {
            if (!ok || i >= n_tiles) return;
            const int s = i & 1;
            if (i >= 2 && !mbar_wait(bar(V_EMPTY + s), ((i >> 1) - 1) & 1, fail_flag)) { ok = false; return; }
            const uint32_t sV = sKV + s * 2 * KV_TILE + KV_TILE;
            mbar_expect_tx(bar(V_FULL + s), KV_TILE);
            for (int sl = 0; sl < SLABS; ++sl)
                tma_load_2d(sV + sl * KV_SLAB, &map_kv, (kv_k_head0 + nkv + kvh) * HD + sl * 64, first + k_first + i * BN,
                            bar(V_FULL + s));
        };
        load_v(0); load_v(1);                          // (Q, K0 and K1 were asked for above)
        load_k(2); load_k(3);
        for (int i = 0; ok && i + 2 < n_tiles; ++i) {
            load_v(i + 2);
            load_k(i + 4);
        }
        if (!ok) atomicExch(&failed, 1);
    } else if (warp == ISSUER_WARP && lane == 0) {
        // ---- the thread that issues the scores: S[it & 1] = Q K(it)^T, two tiles ahead of P V.  (Issuing one
        // tcgen05.mma costs the thread 85 to 110 cycles, more than a product of 64 keys runs: with one thread
        // for both kinds of product, issuing them took 1,900 of a tile's 3,400 cycles.)
        const uint32_t idesc_s = instr_desc(BM, BN, false);
        const uint64_t dQ = smem_desc(sQ), dK[2] = {smem_desc(sKV), smem_desc(sKV + 2 * KV_TILE)};
        bool ok = mbar_wait(bar(Q_FULL), 0, fail_flag);
        for (int it = 0; ok && it < n_tiles; ++it) {
            const int b = it & 1;
            ok = mbar_wait(bar(K_FULL + b), (it >> 1) & 1, fail_flag) &&
                 (it < 2 || mbar_wait(bar(S_EMPTY + b), ((it >> 1) - 1) & 1, fail_flag));
            if (!ok) break;
            fence_after();
            const uint64_t dk = dK[b];
            const uint32_t ts = tS + 64 * b;
#pragma unroll
            for (int sl = 0; sl < SLABS; ++sl)
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    umma(ts, dQ + (uint64_t)((sl * Q_SLAB + kk * 32) >> 4), dk + (uint64_t)((sl * KV_SLAB + kk * 32) >> 4),
                         idesc_s, (sl > 0 || kk > 0) ? 1u : 0u);
            umma_commit(bar(S_FULL + b));             // the scores are there ...
            umma_commit(bar(K_EMPTY + b));            // ... and these keys are no longer needed
        }
        if (!ok) atomicExch(&failed, 1);
    } else if (warp == PV_WARP && lane == 0) {
        // ---- the thread that issues O += P V
        const uint32_t idesc_o = instr_desc(BM, HD, true);
        const uint64_t dV[2] = {smem_desc(sKV + KV_TILE, KV_SLAB), smem_desc(sKV + 2 * KV_TILE + KV_TILE, KV_SLAB)};
        bool ok = true;
        for (int it = 0; ok && it < n_tiles; ++it) {
            const int b = it & 1;
            ok = mbar_wait(bar(P_FULL + b), (it >> 1) & 1, fail_flag) && mbar_wait(bar(V_FULL + b), (it >> 1) & 1, fail_flag);
            if (!ok) break;
            fence_after();
            const uint64_t dv = dV[b];
            const uint32_t tp = tP + 32 * b;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)              // P[:, 16 kk ..] from tensor memory, V[16 kk .., :]: all features in one instruction
                umma_ts(tO, tp + kk * 8, dv + (uint64_t)((kk * 2048) >> 4), idesc_o, (it > 0 || kk > 0) ? 1u : 0u);
            umma_commit(bar(V_EMPTY + b));             // the values are free once these have read them
            umma_commit(bar(O_DONE + b));              // and the accumulator holds tile `it`; P's buffer is free
        }
        if (!ok) atomicExch(&failed, 1);
    } else if (warp < SOFTMAX_WARPS) {
        // ---- softmax: SPLIT threads share query row q0 + r (tensor-memory lane r); this one has keys CPT h .. of
        // each tile and columns OCOLS h .. of the accumulator
        const int quarter = warp & 3, h = warp >> 2;
        const int r = quarter * 32 + lane, row_pos = q0 + r;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const float LOG2E = 1.4426950408889634f;
        // scores in units of log2(e): cap2 tanh(s scale / cap) = cap2 - 2 cap2 / (2^(s k_tanh) + 1), or s scale2
        const float cap2 = cap * LOG2E, scale2 = scale * LOG2E;
        const float k_tanh = CAPPED ? scale / cap * (JANIS_PT_TANH_APPROX ? 1.0f : 2.0f * LOG2E) : 0.f;
        float m_ref = -INFINITY, l_run = 0.f;         // reference of the exponentials (log2 units); sum over this thread's keys
        // Two tiles are in flight in every thread: stage one of tile it + 1 (scores out of tensor memory, scale,
        // cap, masks, this thread's maximum told to the row's other threads) runs before stage two of tile it (the
        // row's maximum, exponentials, P), so that neither the exchange nor the products are waited for.
        // Stage one already subtracts the reference of the exponentials as it stands then (`base`), in the same
        // fused multiply-add that ends the cap; stage two corrects the few tiles whose reference has moved since.
        auto stage_one = [&](int it, uint32_t (&sv)[CPT], float& base) -> bool {
            const int b = it & 1, k0 = k_first + it * BN;
            if (!mbar_wait(bar(S_FULL + b), (it >> 1) & 1, fail_flag)) return false;
            fence_after();
            tmem_ld16(tS + 64 * b + CPT * h + lane_base, sv);
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            fence_before();
            warp_arrive(bar(S_EMPTY + b), lane);      // the scores are in registers
            base = m_ref == -INFINITY ? 0.f : m_ref;
            const float c0 = CAPPED ? cap2 - base : -base, c1 = -2.0f * cap2;
            const bool inner = k0 + BN - 1 <= q0 && k0 + BN <= len && (window <= 0 || k0 > q0 + BM - 1 - window);
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < CPT; ++j) {
                const float s = __uint_as_float(sv[j]);
                float v;
                if (CAPPED) {
#if JANIS_PT_TANH_APPROX
                    v = fmaf(tanh_approx(s * k_tanh), cap2, -base);
#else
                    float rc;
                    asm("rcp.approx.ftz.f32 %0, %1;\n" : "=f"(rc) : "f"(pf::ex2(s * k_tanh) + 1.0f));
                    v = fmaf(rc, c1, c0);              // exact limits: 2^x = inf gives cap2, 2^x = 0 gives -cap2
#endif
                } else {
                    v = fmaf(s, scale2, c0);
                }
                if (!inner) {
                    const int key = k0 + CPT * h + j;
                    const bool seen = key <= row_pos && key < len && (window <= 0 || key > row_pos - window);
                    v = seen ? v : -INFINITY;
                }
                sv[j] = __float_as_uint(v);
                mx = fmaxf(mx, v);
            }
            // (an mbarrier, not bar.sync: a thread that has given up a wait must not leave the others stuck;
            // two of them in turn, since a warp arrives for tile it + 1 before all have arrived for tile it)
            row_max[it & 3][h][r] = mx + base;
            warp_arrive(bar(ROW_X + b), lane);
            return true;
        };
        auto stage_two = [&](int it, uint32_t (&sv)[CPT], float base) -> bool {
            if (!mbar_wait(bar(ROW_X + (it & 1)), (it >> 1) & 1, fail_flag)) return false;
            float mx = row_max[it & 3][0][r];
#pragma unroll
            for (int hh = 1; hh < SPLIT; ++hh) mx = fmaxf(mx, row_max[it & 3][hh][r]);
            // the reference moves only when the maximum has outgrown it by more than RESCALE_STEP
            // (every thread of the row sees the same maximum and decides the same)
            float factor = 1.0f;
            const bool grow = mx > m_ref + RESCALE_STEP || (m_ref == -INFINITY && mx != -INFINITY);
            if (grow) {
                factor = pf::ex2(m_ref - mx);          // 2^(-inf) = 0 the first time
                m_ref = mx;
            }
            const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
            l_run *= factor;
            if (base != m_use) {                       // the reference has moved since stage one of this tile
                const float shift = base - m_use;
#pragma unroll
                for (int j = 0; j < CPT; ++j) sv[j] = __float_as_uint(__uint_as_float(sv[j]) + shift);
            }
            uint32_t pk[CPT / 2];
#pragma unroll
            for (int j = 0; j < CPT; j += 2) {
                const float p0 = pf::ex2(__uint_as_float(sv[j]));
                const float p1 = JANIS_PT_POLY_EX2 ? ex2_poly(__uint_as_float(sv[j + 1])) : pf::ex2(__uint_as_float(sv[j + 1]));
                l_run += p0 + p1;
                pk[j / 2] = pf::pack_bf16(p0, p1);
            }
            // P has two buffers in tensor memory: this tile's is free once the products of the tile before last have
            // finished, so the softmax does not wait for the products of the tile before (it did, with one buffer of
            // P in shared memory: the round trip softmax -> products -> softmax then set the time of a tile, 1.5 us
            // whatever the head size, with the softmax's arithmetic taken out as well as with it).  Only a warp that
            // has to rescale the accumulator waits for them.
            if (it >= 2 && !mbar_wait(bar(O_DONE + (it & 1)), ((it - 2) >> 1) & 1, fail_flag)) return false;
            if (it > 0 && __any_sync(0xffffffffu, grow)) {   // tensor-memory accesses are warp-wide: rows that keep their reference use 1
                if (!mbar_wait(bar(O_DONE + ((it - 1) & 1)), ((it - 1) >> 1) & 1, fail_flag)) return false;
                fence_after();
                {
#pragma unroll 1
                    for (int c = OCOLS * h; c < OCOLS * (h + 1); c += 16) {
                        uint32_t o[16];
                        tmem_ld16(tO + c + lane_base, o);
                        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
                        for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * factor);
                        tmem_st16(tO + c + lane_base, o);
                    }
                    asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
                }
            }
            // The last tile of a sequence that does not end on a tile border: the box of values runs on into rows
            // that are not this sequence's (the next sequence's, padding, whatever the buffer held).  Their
            // columns of P are zero, but 0 x NaN is NaN in the product, so those rows of V are cleared in shared
            // memory once the box has landed (a 128-byte swizzle permutes within a row: whole rows stay whole).
            // Keys of such rows only reach their own columns of S, which the mask replaces.
            {
                const int k0 = k_first + it * BN;
                if (k0 + BN > len) {
                    if (!mbar_wait(bar(V_FULL + (it & 1)), (it >> 1) & 1, fail_flag)) return false;
                    const int n_valid = len - k0;     // >= 1: the tile holds a key that a query of this tile sees
                    unsigned char* v_ptr = smem_raw + (sKV - raw) + (it & 1) * 2 * KV_TILE + KV_TILE;
                    const int pieces = (BN - n_valid) * 8;           // 16-byte pieces per slab
                    for (int idx = threadIdx.x; idx < pieces * SLABS; idx += SOFTMAX_WARPS * 32) {
                        const int sl = idx / pieces, pc = idx % pieces;
                        *reinterpret_cast<uint4*>(v_ptr + sl * KV_SLAB + n_valid * 128 + pc * 16) = make_uint4(0u, 0u, 0u, 0u);
                    }
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");     // before the products read them
                }
            }
            // this thread's CPT keys of row r of P: CPT / 2 columns of its lane in the tile's buffer
            fence_after();
            tmem_st8(tP + 32 * (it & 1) + (CPT / 2) * h + lane_base, pk);
            asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            fence_before();
            warp_arrive(bar(P_FULL + (it & 1)), lane);
            return true;
        };
        uint32_t sv[CPT], sv_next[CPT];
        float base = 0.f, base_next = 0.f;
        bool ok = stage_one(0, sv, base);
        for (int it = 0; ok && it < n_tiles; ++it) {
            if (it + 1 < n_tiles) ok = stage_one(it + 1, sv_next, base_next);
            ok = ok && stage_two(it, sv, base);
#pragma unroll
            for (int j = 0; j < CPT; ++j) sv[j] = sv_next[j];
            base = base_next;
        }
        if (ok) ok = mbar_wait(bar(O_DONE + ((n_tiles - 1) & 1)), ((n_tiles - 1) >> 1) & 1, fail_flag);
        if (!ok) atomicExch(&failed, 1);
        // the row's sum, in the order of the threads' keys
        if (ok) {
            row_sum[h][r] = l_run;                     // exchanged like the maximum of a tile after the last
            warp_arrive(bar(ROW_X + (n_tiles & 1)), lane);
            ok = mbar_wait(bar(ROW_X + (n_tiles & 1)), (n_tiles >> 1) & 1, fail_flag);
            if (!ok) atomicExch(&failed, 1);
        }
        // The tile leaves through shared memory (the rings of keys and values are free now): a thread owns a row
        // of the accumulator, so stores straight from its registers would touch a different row of the output with
        // every lane.  Staged in pieces of 16 bytes, XOR-swizzled by row against bank conflicts, the rows then go
        // out as whole lines.
        unsigned char* stage = smem_raw + (sKV - raw);
        if (ok) {
            fence_after();
            float l_row = 0.f;
#pragma unroll
            for (int hh = 0; hh < SPLIT; ++hh) l_row += row_sum[hh][r];
            if (shared_tile) {
                if (h == 0) {
                    float* prow = partial + ((((size_t)gtile * nq + head) * parts + part) * BM + r) * pf::PART_ROW;
                    prow[0] = m_ref;
                    prow[1] = l_row;
                }
#pragma unroll 1
                for (int c = OCOLS * h; c < OCOLS * (h + 1); c += 16) {
                    uint32_t o[16];
                    tmem_ld16(tO + c + lane_base, o);
                    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 16; j += 4)
                        *reinterpret_cast<uint4*>(stage + (size_t)r * (HD * 4) + ((((c + j) >> 2) ^ (r & 7)) << 4)) =
                            make_uint4(o[j], o[j + 1], o[j + 2], o[j + 3]);
                }
            } else {
                const float inv = 1.0f / l_row;
#pragma unroll 1
                for (int c = OCOLS * h; c < OCOLS * (h + 1); c += 16) {
                    uint32_t o[16];
                    tmem_ld16(tO + c + lane_base, o);
                    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 16; j += 8) {
                        uint4 w;
                        w.x = pf::pack_bf16(__uint_as_float(o[j]) * inv, __uint_as_float(o[j + 1]) * inv);
                        w.y = pf::pack_bf16(__uint_as_float(o[j + 2]) * inv, __uint_as_float(o[j + 3]) * inv);
                        w.z = pf::pack_bf16(__uint_as_float(o[j + 4]) * inv, __uint_as_float(o[j + 5]) * inv);
                        w.w = pf::pack_bf16(__uint_as_float(o[j + 6]) * inv, __uint_as_float(o[j + 7]) * inv);
                        *reinterpret_cast<uint4*>(stage + (size_t)r * (HD * 2) + ((((c + j) >> 3) ^ (r & 7)) << 4)) = w;
                    }
                }
            }
            // all rows are staged (the exchange barrier once more, as for a tile after the sums)
            warp_arrive(bar(ROW_X + ((n_tiles + 1) & 1)), lane);
            ok = mbar_wait(bar(ROW_X + ((n_tiles + 1) & 1)), ((n_tiles + 1) >> 1) & 1, fail_flag);
            if (!ok) atomicExch(&failed, 1);
        }
        if (ok) {
            const int rows = min(BM, len - q0);
            if (shared_tile) {
                constexpr int PIECES = HD / 4;        // pieces of 4 floats in a row
                float* pbase = partial + (((size_t)gtile * nq + head) * parts + part) * BM * pf::PART_ROW;
                for (int idx = threadIdx.x; idx < rows * PIECES; idx += SOFTMAX_WARPS * 32) {
                    const int rr = idx / PIECES, pc = idx % PIECES;
                    const uint4 v = *reinterpret_cast<const uint4*>(stage + (size_t)rr * (HD * 4) + ((pc ^ (rr & 7)) << 4));
                    float* dst = pbase + (size_t)rr * pf::PART_ROW + 2 + pc * 4;    // 8-byte aligned
                    *reinterpret_cast<uint2*>(dst) = make_uint2(v.x, v.y);
                    *reinterpret_cast<uint2*>(dst + 2) = make_uint2(v.z, v.w);
                }
            } else {
                constexpr int PIECES = HD / 8;        // pieces of 8 bfloat16 in a row
                bf16* obase = out + (size_t)(first + q0) * nq * HD + (size_t)head * HD;
                for (int idx = threadIdx.x; idx < rows * PIECES; idx += SOFTMAX_WARPS * 32) {
                    const int rr = idx / PIECES, pc = idx % PIECES;
                    *reinterpret_cast<uint4*>(obase + (size_t)rr * nq * HD + pc * 8) =
                        *reinterpret_cast<const uint4*>(stage + (size_t)rr * (HD * 2) + ((pc ^ (rr & 7)) << 4));
                }
            }
        }
    }
    __syncwarp();
    fence_before();
    __syncthreads();
    if (warp == ISSUER_WARP)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    if (failed && threadIdx.x == 0) atomicAdd(&g_timeouts, 1);
}

// ---------------------------------------------------------------------------------------------------------------
// The same work by CTAs that stay: one CTA an SM takes item after item (a tile of queries of one head, or a part of
// one) from a counter, so that what a CTA costs besides its tiles is paid once, not per tile of queries: the launch
// of a CTA of this size and its way out (2 to 3 us), Q and the first keys (asked for while the item before is still
// at its last tiles), the products' start.  What stays per item is the way out of its result.  An item's place is
// told to the other roles through two slots in shared memory; the rings of keys and values, the two score buffers,
// P and the accumulator carry on from item to item (their barriers count tiles across items).  The result leaves
// through the ring stage of the item's last tile (bfloat16: one stage holds a tile of queries), which is the stage
// of the next item's second tile: the loader brings the next item's first tile meanwhile and waits for the way out
// before the second; a partial result (float) takes both stages, and the loader waits before the first.
// ---------------------------------------------------------------------------------------------------------------
struct Item {
    int seq, q0, len, first, k_first, n_tiles, head, gtile, part, np;   // n_tiles < 0: there is no further item
};

enum { ITEM_FULL = N_BARS, ITEM_EMPTY = N_BARS + 2, Q_EMPTY = N_BARS + 4, EPI_DONE = N_BARS + 5, N_BARS_ITEMS = N_BARS + 6 };

// A launch's counters: the next item, and the CTAs that have left (the last one puts both back to 0).  Launches
// take the slots in turn, so that launches in flight together (other streams) do not share one; SCHED_SLOTS of
// them at once is the limit of that.
constexpr int SCHED_SLOTS = 64;
__device__ int g_sched[SCHED_SLOTS][2];

// find_tile by a whole warp: 32 sequences a round
__device__ __forceinline__ bool find_tile_warp(int tile, const int* __restrict__ seq_len, int n_seq, int lane, int& seq,
                                               int& q0, int& len) {
    int before = 0;
    for (int s0 = 0; s0 < n_seq; s0 += 32) {
        const int n = s0 + lane < n_seq ? seq_len[s0 + lane] : 0;
        const int nt = (n + BM - 1) / BM;
        int incl = nt;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += v;
        }
        const int lo = before + incl - nt;
        const unsigned hit = __ballot_sync(0xffffffffu, tile >= lo && tile < lo + nt);
        if (hit) {
            const int src = __ffs(hit) - 1;
            seq = s0 + src;
            q0 = (tile - __shfl_sync(0xffffffffu, lo, src)) * BM;
            len = __shfl_sync(0xffffffffu, n, src);
            return true;
        }
        before += __shfl_sync(0xffffffffu, incl, 31);
    }
    return false;
}

template <bool CAPPED>
__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tc05_items_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                               const int* __restrict__ seq_first_row, const int* __restrict__ seq_len, int n_seq,
                               bf16* __restrict__ out, int nq, int nkv, int kv_k_head0, float scale, float cap, int window,
                               int parts, int piece, float* __restrict__ partial, int n_places, int sched_slot) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[N_BARS_ITEMS];
    int* sched = g_sched[sched_slot];
    __shared__ uint32_t tmem_slot;
    __shared__ int failed;
    __shared__ float row_max[4][SPLIT][BM];
    __shared__ float row_sum[SPLIT][BM];
    __shared__ Item items[2];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t raw = (uint32_t)__cvta_generic_to_shared(smem_raw);
    const uint32_t sQ = (raw + 1023) & ~1023u;
    const uint32_t sKV = sQ + Q_BYTES;
    const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(bars);
    auto bar = [&](int i) { return bar0 + 8 * i; };
    const volatile int* fail_flag = &failed;

    if (warp == LOADER_WARP && lane == 0) {
        mbar_init(bar(Q_FULL), 1);
        mbar_init(bar(Q_EMPTY), 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar(K_FULL + i), 1);
            mbar_init(bar(K_EMPTY + i), 1);
            mbar_init(bar(V_FULL + i), 1);
            mbar_init(bar(V_EMPTY + i), 1);
            mbar_init(bar(S_FULL + i), 1);
            mbar_init(bar(S_EMPTY + i), SOFTMAX_WARPS);
            mbar_init(bar(ROW_X + i), SOFTMAX_WARPS);
            mbar_init(bar(ITEM_FULL + i), 1);
            mbar_init(bar(ITEM_EMPTY + i), SOFTMAX_WARPS + 2);
            mbar_init(bar(P_FULL + i), SOFTMAX_WARPS);
            mbar_init(bar(O_DONE + i), 1);
        }
        mbar_init(bar(EPI_DONE), SOFTMAX_WARPS);
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == ISSUER_WARP) {
        const uint32_t slot = (uint32_t)__cvta_generic_to_shared(&tmem_slot);
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(slot), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    grid_dependents_launch();

    // The next item from the counter, by the whole loader warp (the step's tables were written before the kernel
    // ahead of this one started, and the counter is this kernel's own: the items are found before the wait).
    const int total = n_places * nq;
    auto fetch = [&]() -> Item {
        Item it;
        it.n_tiles = -1;
        it.seq = it.q0 = it.len = it.first = it.k_first = it.head = it.gtile = it.part = it.np = 0;
        for (;;) {
            int idx = 0;
            if (lane == 0) idx = atomicAdd(&sched[0], 1);
            idx = __shfl_sync(0xffffffffu, idx, 0);
            if (idx >= total) return it;
            const int place = n_places - 1 - idx / nq;     // heads vary fastest; the last tile of queries comes first
            const int gtile = place / parts, part = place % parts;
            int seq = 0, q0 = 0, len = 0;
            if (!find_tile_warp(gtile, seq_len, n_seq, lane, seq, q0, len)) continue;
            int k_first, n_tiles;
            pf::key_tiles(q0, len, window, k_first, n_tiles);
            const int np = pf::parts_of(n_tiles, parts, piece);
            if (part >= np) continue;
            if (np > 1) {
                const int t0 = (int)((long long)n_tiles * part / np), t1 = (int)((long long)n_tiles * (part + 1) / np);
                k_first += t0 * BN;
                n_tiles = t1 - t0;
            }
            it.seq = seq; it.q0 = q0; it.len = len; it.first = seq_first_row[seq]; it.k_first = k_first;
            it.n_tiles = n_tiles; it.head = idx % nq; it.gtile = gtile; it.part = part; it.np = np;
            return it;
        }
    };
    // item number k goes into slot k & 1 once the roles have taken item k - 2 out of it
    auto publish = [&](int k, const Item& it) -> bool {
        if (k >= 2 && !mbar_wait(bar(ITEM_EMPTY + (k & 1)), ((k >> 1) - 1) & 1, fail_flag)) return false;
        items[k & 1] = it;
        mbar_arrive(bar(ITEM_FULL + (k & 1)));
        return true;
    };
    Item cur;
    cur.n_tiles = -1;
    if (warp == LOADER_WARP) {
        cur = fetch();
        if (lane == 0) publish(0, cur);
    }
    grid_dependency_wait();
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = tmem_slot;
    const uint32_t tO = tmem, tS = tmem + HD, tP = tS + 128;
    const int group = nq / nkv;

    if (warp == LOADER_WARP) {
        // ---- loader
        bool ok = true;
        int g = 0, prev_np = 1;                      // tiles before this item; parts of the item before
        for (int k = 0; cur.n_tiles >= 0; ++k) {
            const int n = cur.n_tiles, kvh = cur.head / group;
            if (lane == 0) {
                // (Q is free: the item before was taken only after its last scores, below)
                mbar_expect_tx(bar(Q_FULL), Q_BYTES);
                for (int sl = 0; sl < SLABS; ++sl)
                    tma_load_2d(sQ + sl * Q_SLAB, &map_q, cur.head * HD + sl * 64, cur.first + cur.q0, bar(Q_FULL));
                auto load_k = [&](int i) {
                    if (!ok || i >= n) return;
                    const int gi = g + i, s = gi & 1;
                    if (gi >= 2 && !mbar_wait(bar(K_EMPTY + s), ((gi >> 1) - 1) & 1, fail_flag)) { ok = false; return; }
                    const uint32_t sK = sKV + s * 2 * KV_TILE;
                    mbar_expect_tx(bar(K_FULL + s), KV_TILE);
                    for (int sl = 0; sl < SLABS; ++sl)
                        tma_load_2d(sK + sl * KV_SLAB, &map_kv, (kv_k_head0 + kvh) * HD + sl * 64,
                                    cur.first + cur.k_first + i * BN, bar(K_FULL + s));
                };
                auto load_v = [&](int i) {
                    if (!ok || i >= n) return;
                    const int gi = g + i, s = gi & 1;
                    if (gi >= 2 && !mbar_wait(bar(V_EMPTY + s), ((gi >> 1) - 1) & 1, fail_flag)) { ok = false; return; }
                    const uint32_t sV = sKV + s * 2 * KV_TILE + KV_TILE;
                    mbar_expect_tx(bar(V_FULL + s), KV_TILE);
                    for (int sl = 0; sl < SLABS; ++sl)
                        tma_load_2d(sV + sl * KV_SLAB, &map_kv, (kv_k_head0 + nkv + kvh) * HD + sl * 64,
                                    cur.first + cur.k_first + i * BN, bar(V_FULL + s));
                };
                // the item before leaves through the stage of this item's second tile (both stages, if it leaves a
                // partial result): every item's way out is waited for once, in order
                auto way_out = [&]() {
                    if (ok && k > 0) ok = mbar_wait(bar(EPI_DONE), (k - 1) & 1, fail_flag);
                };
                if (prev_np > 1) way_out();
                load_k(0); load_v(0);
                if (prev_np <= 1) way_out();
                load_k(1); load_v(1);
                load_k(2); load_k(3);
                for (int i = 0; ok && i + 2 < n; ++i) {
                    load_v(i + 2);
                    load_k(i + 4);
                }
                // The next item is taken late, when this item's last scores are done (two tiles and the way out are
                // left): a CTA that took its next item early would hold it while other CTAs have nothing to do.
                if (ok) ok = mbar_wait(bar(Q_EMPTY), k & 1, fail_flag);
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            const Item nxt = fetch();
            if (lane == 0) ok = publish(k + 1, nxt);
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            g += n;
            prev_np = cur.np;
            cur = nxt;
        }
        if (!ok && lane == 0) atomicExch(&failed, 1);
    } else if (warp == ISSUER_WARP && lane == 0) {
        // ---- the thread that issues the scores
        const uint32_t idesc_s = instr_desc(BM, BN, false);
        const uint64_t dQ = smem_desc(sQ), dK[2] = {smem_desc(sKV), smem_desc(sKV + 2 * KV_TILE)};
        bool ok = true;
        int g = 0;
        for (int k = 0; ok; ++k) {
            ok = mbar_wait(bar(ITEM_FULL + (k & 1)), (k >> 1) & 1, fail_flag);
            if (!ok) break;
            const int n = items[k & 1].n_tiles;
            mbar_arrive(bar(ITEM_EMPTY + (k & 1)));
            if (n < 0) break;
            ok = mbar_wait(bar(Q_FULL), k & 1, fail_flag);
            for (int i = 0; ok && i < n; ++i) {      // S[(g + i) & 1] = Q K(i)^T
                const int gi = g + i, b = gi & 1;
                ok = mbar_wait(bar(K_FULL + b), (gi >> 1) & 1, fail_flag) &&
                     (gi < 2 || mbar_wait(bar(S_EMPTY + b), ((gi >> 1) - 1) & 1, fail_flag));
                if (!ok) break;
                fence_after();
                const uint64_t dk = dK[b];
                const uint32_t ts = tS + 64 * b;
#pragma unroll
                for (int sl = 0; sl < SLABS; ++sl)
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        umma(ts, dQ + (uint64_t)((sl * Q_SLAB + kk * 32) >> 4), dk + (uint64_t)((sl * KV_SLAB + kk * 32) >> 4),
                             idesc_s, (sl > 0 || kk > 0) ? 1u : 0u);
                umma_commit(bar(S_FULL + b));
                umma_commit(bar(K_EMPTY + b));
                if (i == n - 1) umma_commit(bar(Q_EMPTY));     // the item's last scores: Q may be overwritten
            }
            g += n;
        }
        if (!ok) atomicExch(&failed, 1);
    } else if (warp == PV_WARP && lane == 0) {
        // ---- the thread that issues O += P V
        const uint32_t idesc_o = instr_desc(BM, HD, true);
        const uint64_t dV[2] = {smem_desc(sKV + KV_TILE, KV_SLAB), smem_desc(sKV + 2 * KV_TILE + KV_TILE, KV_SLAB)};
        bool ok = true;
        int g = 0;
        for (int k = 0; ok; ++k) {
            ok = mbar_wait(bar(ITEM_FULL + (k & 1)), (k >> 1) & 1, fail_flag);
            if (!ok) break;
            const int n = items[k & 1].n_tiles;
            mbar_arrive(bar(ITEM_EMPTY + (k & 1)));
            if (n < 0) break;
            for (int it = 0; ok && it < n; ++it) {
                const int gi = g + it, b = gi & 1;
                ok = mbar_wait(bar(P_FULL + b), (gi >> 1) & 1, fail_flag) && mbar_wait(bar(V_FULL + b), (gi >> 1) & 1, fail_flag);
                if (!ok) break;
                fence_after();
                const uint64_t dv = dV[b];
                const uint32_t tp = tP + 32 * b;
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    umma_ts(tO, tp + kk * 8, dv + (uint64_t)((kk * 2048) >> 4), idesc_o, (it > 0 || kk > 0) ? 1u : 0u);
                umma_commit(bar(V_EMPTY + b));
                umma_commit(bar(O_DONE + b));
            }
            g += n;
        }
        if (!ok) atomicExch(&failed, 1);
    } else if (warp < SOFTMAX_WARPS) {
        // ---- softmax (see the kernel above; the barriers of tiles count on from item to item)
        const int quarter = warp & 3, h = warp >> 2;
        const int r = quarter * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const float LOG2E = 1.4426950408889634f;
        const float cap2 = cap * LOG2E, scale2 = scale * LOG2E;
        const float k_tanh = CAPPED ? scale / cap * (JANIS_PT_TANH_APPROX ? 1.0f : 2.0f * LOG2E) : 0.f;
        bool ok = true;
        int g = 0, gx = 0;                           // tiles, and exchanges through ROW_X, before this item
        for (int k = 0; ok; ++k) {
            ok = mbar_wait(bar(ITEM_FULL + (k & 1)), (k >> 1) & 1, fail_flag);
            if (!ok) break;
            const Item me = items[k & 1];
            warp_arrive(bar(ITEM_EMPTY + (k & 1)), lane);
            if (me.n_tiles < 0) break;
            const int n_tiles = me.n_tiles, q0 = me.q0, len = me.len, k_first = me.k_first;
            const int row_pos = q0 + r;
            const bool shared_tile = me.np > 1;
            float m_ref = -INFINITY, l_run = 0.f;
            auto stage_one = [&](int it, uint32_t (&sv)[CPT], float& base) -> bool {
                const int gi = g + it, x = gx + it, b = gi & 1, k0 = k_first + it * BN;
                if (!mbar_wait(bar(S_FULL + b), (gi >> 1) & 1, fail_flag)) return false;
                fence_after();
                tmem_ld16(tS + 64 * b + CPT * h + lane_base, sv);
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                fence_before();
                warp_arrive(bar(S_EMPTY + b), lane);
                base = m_ref == -INFINITY ? 0.f : m_ref;
                const float c0 = CAPPED ? cap2 - base : -base, c1 = -2.0f * cap2;
                const bool inner = k0 + BN - 1 <= q0 && k0 + BN <= len && (window <= 0 || k0 > q0 + BM - 1 - window);
                float mx = -INFINITY;
#pragma unroll
                for (int j = 0; j < CPT; ++j) {
                    const float s = __uint_as_float(sv[j]);
                    float v;
                    if (CAPPED) {
#if JANIS_PT_TANH_APPROX
                        v = fmaf(tanh_approx(s * k_tanh), cap2, -base);
#else
                        float rc;
                        asm("rcp.approx.ftz.f32 %0, %1;\n" : "=f"(rc) : "f"(pf::ex2(s * k_tanh) + 1.0f));
                        v = fmaf(rc, c1, c0);
#endif
                    } else {
                        v = fmaf(s, scale2, c0);
                    }
                    if (!inner) {
                        const int key = k0 + CPT * h + j;
                        const bool seen = key <= row_pos && key < len && (window <= 0 || key > row_pos - window);
                        v = seen ? v : -INFINITY;
                    }
                    sv[j] = __float_as_uint(v);
                    mx = fmaxf(mx, v);
                }
                row_max[x & 3][h][r] = mx + base;
                warp_arrive(bar(ROW_X + (x & 1)), lane);
                return true;
            };
            auto stage_two = [&](int it, uint32_t (&sv)[CPT], float base) -> bool {
                const int gi = g + it, x = gx + it, b = gi & 1;
                if (!mbar_wait(bar(ROW_X + (x & 1)), (x >> 1) & 1, fail_flag)) return false;
                float mx = row_max[x & 3][0][r];
#pragma unroll
                for (int hh = 1; hh < SPLIT; ++hh) mx = fmaxf(mx, row_max[x & 3][hh][r]);
                float factor = 1.0f;
                const bool grow = mx > m_ref + RESCALE_STEP || (m_ref == -INFINITY && mx != -INFINITY);
                if (grow) {
                    factor = pf::ex2(m_ref - mx);
                    m_ref = mx;
                }
                const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
                l_run *= factor;
                if (base != m_use) {
                    const float shift = base - m_use;
#pragma unroll
                    for (int j = 0; j < CPT; ++j) sv[j] = __float_as_uint(__uint_as_float(sv[j]) + shift);
                }
                uint32_t pk[CPT / 2];
#pragma unroll
                for (int j = 0; j < CPT; j += 2) {
                    const float p0 = pf::ex2(__uint_as_float(sv[j]));
                    const float p1 = JANIS_PT_POLY_EX2 ? ex2_poly(__uint_as_float(sv[j + 1])) : pf::ex2(__uint_as_float(sv[j + 1]));
                    l_run += p0 + p1;
                    pk[j / 2] = pf::pack_bf16(p0, p1);
                }
                // P's buffer is free once the products of the tile before last have finished (across items too); only
                // a warp that has to rescale the accumulator waits for the products of the tile before
                if (gi >= 2 && !mbar_wait(bar(O_DONE + b), ((gi - 2) >> 1) & 1, fail_flag)) return false;
                if (it > 0 && __any_sync(0xffffffffu, grow)) {
                    if (!mbar_wait(bar(O_DONE + ((gi - 1) & 1)), ((gi - 1) >> 1) & 1, fail_flag)) return false;
                    fence_after();
                    {
#pragma unroll 1
                        for (int c = OCOLS * h; c < OCOLS * (h + 1); c += 16) {
                            uint32_t o[16];
                            tmem_ld16(tO + c + lane_base, o);
                            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
                            for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * factor);
                            tmem_st16(tO + c + lane_base, o);
                        }
                        asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
                    }
                }
                {   // rows of the last box of values beyond the sequence's end are cleared (see the kernel above)
                    const int k0 = k_first + it * BN;
                    if (k0 + BN > len) {
                        if (!mbar_wait(bar(V_FULL + b), (gi >> 1) & 1, fail_flag)) return false;
                        const int n_valid = len - k0;
                        unsigned char* v_ptr = smem_raw + (sKV - raw) + b * 2 * KV_TILE + KV_TILE;
                        const int pieces = (BN - n_valid) * 8;
                        for (int idx = threadIdx.x; idx < pieces * SLABS; idx += SOFTMAX_WARPS * 32) {
                            const int sl = idx / pieces, pc = idx % pieces;
                            *reinterpret_cast<uint4*>(v_ptr + sl * KV_SLAB + n_valid * 128 + pc * 16) = make_uint4(0u, 0u, 0u, 0u);
                        }
                        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");     // before the products read them
                    }
                }
                fence_after();
                tmem_st8(tP + 32 * b + (CPT / 2) * h + lane_base, pk);
                asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
                fence_before();
                warp_arrive(bar(P_FULL + b), lane);
                return true;
            };
            uint32_t sv[CPT], sv_next[CPT];
            float base = 0.f, base_next = 0.f;
            ok = stage_one(0, sv, base);
            for (int it = 0; ok && it < n_tiles; ++it) {
                if (it + 1 < n_tiles) ok = stage_one(it + 1, sv_next, base_next);
                ok = ok && stage_two(it, sv, base);
#pragma unroll
                for (int j = 0; j < CPT; ++j) sv[j] = sv_next[j];
                base = base_next;
            }
            if (ok) ok = mbar_wait(bar(O_DONE + ((g + n_tiles - 1) & 1)), ((g + n_tiles - 1) >> 1) & 1, fail_flag);
            if (ok) {
                const int x = gx + n_tiles;
                row_sum[h][r] = l_run;
                warp_arrive(bar(ROW_X + (x & 1)), lane);
                ok = mbar_wait(bar(ROW_X + (x & 1)), (x >> 1) & 1, fail_flag);
            }
            // the way out: through the stage of the item's last tile (a partial result: through both stages)
            unsigned char* stage = smem_raw + (sKV - raw) + (shared_tile ? 0 : ((g + n_tiles - 1) & 1) * 2 * KV_TILE);
            if (ok) {
                fence_after();
                float l_row = 0.f;
#pragma unroll
                for (int hh = 0; hh < SPLIT; ++hh) l_row += row_sum[hh][r];
                if (shared_tile) {
                    if (h == 0) {
                        float* prow = partial + ((((size_t)me.gtile * nq + me.head) * parts + me.part) * BM + r) * pf::PART_ROW;
                        prow[0] = m_ref;
                        prow[1] = l_row;
                    }
#pragma unroll 1
                    for (int c = OCOLS * h; c < OCOLS * (h + 1); c += 16) {
                        uint32_t o[16];
                        tmem_ld16(tO + c + lane_base, o);
                        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
                        for (int j = 0; j < 16; j += 4)
                            *reinterpret_cast<uint4*>(stage + (size_t)r * (HD * 4) + ((((c + j) >> 2) ^ (r & 7)) << 4)) =
                                make_uint4(o[j], o[j + 1], o[j + 2], o[j + 3]);
                    }
                } else {
                    const float inv = 1.0f / l_row;
#pragma unroll 1
                    for (int c = OCOLS * h; c < OCOLS * (h + 1); c += 16) {
                        uint32_t o[16];
                        tmem_ld16(tO + c + lane_base, o);
                        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
                        for (int j = 0; j < 16; j += 8) {
                            uint4 w;
                            w.x = pf::pack_bf16(__uint_as_float(o[j]) * inv, __uint_as_float(o[j + 1]) * inv);
                            w.y = pf::pack_bf16(__uint_as_float(o[j + 2]) * inv, __uint_as_float(o[j + 3]) * inv);
                            w.z = pf::pack_bf16(__uint_as_float(o[j + 4]) * inv, __uint_as_float(o[j + 5]) * inv);
                            w.w = pf::pack_bf16(__uint_as_float(o[j + 6]) * inv, __uint_as_float(o[j + 7]) * inv);
                            *reinterpret_cast<uint4*>(stage + (size_t)r * (HD * 2) + ((((c + j) >> 3) ^ (r & 7)) << 4)) = w;
                        }
                    }
                }
                fence_before();                       // the accumulator has been read: the next item's products may overwrite it
                const int x = gx + n_tiles + 1;
                warp_arrive(bar(ROW_X + (x & 1)), lane);
                ok = mbar_wait(bar(ROW_X + (x & 1)), (x >> 1) & 1, fail_flag);
            }
            if (ok) {
                const int rows = min(BM, len - q0);
                if (shared_tile) {
                    constexpr int PIECES = HD / 4;
                    float* pbase = partial + (((size_t)me.gtile * nq + me.head) * parts + me.part) * BM * pf::PART_ROW;
                    for (int idx = threadIdx.x; idx < rows * PIECES; idx += SOFTMAX_WARPS * 32) {
                        const int rr = idx / PIECES, pc = idx % PIECES;
                        const uint4 v = *reinterpret_cast<const uint4*>(stage + (size_t)rr * (HD * 4) + ((pc ^ (rr & 7)) << 4));
                        float* dst = pbase + (size_t)rr * pf::PART_ROW + 2 + pc * 4;
                        *reinterpret_cast<uint2*>(dst) = make_uint2(v.x, v.y);
                        *reinterpret_cast<uint2*>(dst + 2) = make_uint2(v.z, v.w);
                    }
                } else {
                    constexpr int PIECES = HD / 8;
                    bf16* obase = out + (size_t)(me.first + q0) * nq * HD + (size_t)me.head * HD;
                    for (int idx = threadIdx.x; idx < rows * PIECES; idx += SOFTMAX_WARPS * 32) {
                        const int rr = idx / PIECES, pc = idx % PIECES;
                        *reinterpret_cast<uint4*>(obase + (size_t)rr * nq * HD + pc * 8) =
                            *reinterpret_cast<const uint4*>(stage + (size_t)rr * (HD * 2) + ((pc ^ (rr & 7)) << 4));
                    }
                }
                // the stage has been read (generic proxy) before the loader's bulk copies (async proxy) overwrite it
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                warp_arrive(bar(EPI_DONE), lane);
            }
            g += n_tiles;
            gx += n_tiles + 2;
        }
        if (!ok) atomicExch(&failed, 1);
    }
    __syncwarp();
    fence_before();
    __syncthreads();
    if (warp == ISSUER_WARP)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    if (threadIdx.x == 0) {
        if (failed) atomicAdd(&g_timeouts, 1);
        // the last CTA to leave puts the counters back for the next launch
        __threadfence();
        if (atomicAdd(&sched[1], 1) == (int)gridDim.x - 1) {
            sched[0] = 0;
            sched[1] = 0;
            __threadfence();
        }
    }
}

// ---- host side: tensor maps over the packed rows
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

// a [rows, cols] bfloat16 matrix, cols contiguous, in boxes of 64 x box_rows with the 128-byte swizzle
static bool make_map(CUtensorMap* map, const void* ptr, int rows, int cols, int box_rows) {
    EncodeTiled enc = encoder();
    if (!enc) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace pt

// Which form of the kernel a step runs: 0 a CTA per tile of queries and head, 2 CTAs that stay and take item after
// item, 1 (default) by the step's size: the CTAs that stay where the step has a place an SM or more (they save the
// coming and going of a CTA, about 3 us an item, and ask for their next item late, so that none holds work that
// another could do), a CTA per tile below that (there the two are equal).  Measured per layer at 8 heads of 256, a
// CTA per tile against CTAs that stay: 4 prompts of 4,096 tokens 357 -> 320 us, one of 8,192 321 -> 301, one of
// 4,096 95.8 -> 91.3, 40 of 100 tokens 30.8 -> 24.4, one of 2,048 40.2 = 40.2, two of 1,024 29.3 -> 30.2.
static int g_tc05_items = 1;

static int tc05_sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
    }
    return n;
}

int launch_prefill_tc05(const void* q_src, const void* kv_src, int n_tok, const int* seq_first_row, const int* seq_len,
                        int n_seq, int n_tiles_bound, void* out, int nq, int nkv, int q_row_heads, int kv_row_heads,
                        int kv_k_head0, float scale, float cap, int window, int parts, int piece, float* partial,
                        cudaStream_t stream) {
    if (!pt::SUPPORTED) return -1;
    CUtensorMap mq, mkv;
    if (!pt::make_map(&mq, q_src, n_tok, q_row_heads * pt::HD, pt::BM) ||
        !pt::make_map(&mkv, kv_src, n_tok, kv_row_heads * pt::HD, pt::BN))
        return -1;                                    // no encoder, or operands it refuses: the other kernel runs
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(pt::attn_prefill_tc05_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             pt::SMEM_BYTES);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(pt::attn_prefill_tc05_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     pt::SMEM_BYTES);
        if (e != cudaSuccess) return fail("attn_prefill_tc05: shared memory of %d bytes refused: %s", pt::SMEM_BYTES,
                                          cudaGetErrorString(e));
        configured = true;
    }
    const bool many = (long long)n_tiles_bound * parts * nq >= (long long)tc05_sm_count();
    if (g_tc05_items == 2 || (g_tc05_items == 1 && many)) {
        static bool items_configured = false;
        if (!items_configured) {
            cudaError_t e = cudaFuncSetAttribute(pt::attn_prefill_tc05_items_kernel<true>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, pt::SMEM_BYTES);
            if (e == cudaSuccess)
                e = cudaFuncSetAttribute(pt::attn_prefill_tc05_items_kernel<false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, pt::SMEM_BYTES);
            if (e != cudaSuccess) return fail("attn_prefill_tc05: shared memory of %d bytes refused: %s", pt::SMEM_BYTES,
                                              cudaGetErrorString(e));
            items_configured = true;
        }
        static int next_slot = 0;
        const int slot = next_slot;
        next_slot = (next_slot + 1) % pt::SCHED_SLOTS;
        const int n_places = n_tiles_bound * parts;
        const long long total = (long long)n_places * nq;
        const int ctas = (int)std::min<long long>(total, tc05_sm_count());
        auto items = cap > 0.f ? pt::attn_prefill_tc05_items_kernel<true> : pt::attn_prefill_tc05_items_kernel<false>;
        return launch_kernel("attn_prefill_tc05", items, dim3(ctas), dim3(pt::THREADS), pt::SMEM_BYTES, stream, 1, mq, mkv,
                             seq_first_row, seq_len, n_seq, (bf16*)out, nq, nkv, kv_k_head0, scale, cap, window, parts,
                             piece, partial, n_places, slot);
    }
    auto kernel = cap > 0.f ? pt::attn_prefill_tc05_kernel<true> : pt::attn_prefill_tc05_kernel<false>;
    return launch_kernel("attn_prefill_tc05", kernel, dim3(nq, n_tiles_bound * parts), dim3(pt::THREADS), pt::SMEM_BYTES,
                         stream, 1, mq, mkv, seq_first_row, seq_len, n_seq, (bf16*)out, nq, nkv, kv_k_head0, scale, cap,
                         window, parts, piece, partial);
}

int prefill_tc05_timeouts_async(int* host, cudaStream_t stream) {
    cudaError_t e = cudaMemcpyFromSymbolAsync(host, pt::g_timeouts, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
    return e == cudaSuccess ? 0 : fail("attn_timeouts_async: %s", cudaGetErrorString(e));
}

}  // namespace janis

// How often a CTA of the tcgen05 prompt kernel has given up a wait since the library was loaded (0 unless
// something is badly wrong).  Synchronises the device.
JANIS_EXPORT int janis_attn_tc05_timeouts() {
    int n = -1;
    if (cudaMemcpyFromSymbol(&n, janis::pt::g_timeouts, sizeof(int)) != cudaSuccess) return -1;
    return n;
}

// Which form of the tcgen05 prompt kernel runs: 0 = a CTA per tile of queries and head, 2 = CTAs that stay and take
// item after item, 1 = chosen by the step's size (the default).  All give the same results.
JANIS_EXPORT void janis_attn_set_prefill_items(int how) { janis::g_tc05_items = how < 0 || how > 2 ? 1 : how; }
