// Prompt attention in bfloat16 on the tensor cores (mma.sync.m16n8k16, float
// accumulation), one head size per compiled library (JANIS_HEAD_DIM).
//
// Packed sequences of unequal lengths.  They start at position 0, or (template flag EXT) go on from what
// earlier steps stored: the keys and values of those positions are then read from the paged cache line, row by
// row, the step's own from the step's buffer.  One CTA owns BM
// consecutive queries of one sequence and one query head: each of its warps holds 16
// query rows, walks the key tiles of 64 that the causal mask and the window leave,
// and keeps the running maximum, the running sum and the unnormalised output in
// registers (online softmax).  Keys and values of the next tile are copied into the
// other half of a double buffer (cp.async) while the tensor cores work on this one.
// Per tile: S = Q K^T from shared memory (ldmatrix), s * scale, cap * tanh(s / cap),
// mask on absolute positions, exp, P rounded to bfloat16 as the left operand of P V.
//
// tanh and exp here are built on ex2.approx and rcp.approx: tanh(x) = 1 - 2 / (e^2x + 1)
// has an absolute error near 2e-7, far below the rounding of P to bfloat16 that
// follows; a score needs about 14 instructions instead of about 50 with tanhf and
// expf, which had made the softmax, not the products, the kernel's main cost.  The
// float32 path of the library does not use this kernel.
// Shared-memory rows are XOR-swizzled in 16-byte pieces against ldmatrix bank conflicts.
//
// A prompt step with few tiles of queries (a short prompt, few heads) leaves SMs idle, and its last tile
// walks all the keys while the first walks one tile of them.  Such a step cuts the key tiles of a tile of
// queries into pieces of at most `piece` tiles (no more than `parts` = 4 pieces): each piece is one CTA's, which
// writes its maximum, sum and unnormalised output to scratch, and a second kernel adds the pieces.
#include <algorithm>
#include <functional>
#include <map>
#include <mutex>
#include <queue>
#include <tuple>
#include <vector>

#include "attention_prefill_tiles.cuh"

namespace janis {
namespace pf {

constexpr int THREADS = WARPS * 32;
constexpr int CHUNKS = HD / 8;                        // 16-byte pieces per row
constexpr int swz_pow2(int n) { return n % 8 == 0 ? 8 : (n % 4 == 0 ? 4 : (n % 2 == 0 ? 2 : 1)); }
constexpr int SWZ_MASK = swz_pow2(CHUNKS) - 1;
constexpr int ROW_BYTES = HD * 2;
constexpr int Q_BYTES = BM * ROW_BYTES;
constexpr int KV_BYTES = BN * ROW_BYTES;              // one of K or V, one stage
constexpr int SMEM_BYTES = Q_BYTES + 4 * KV_BYTES;    // Q, then two stages of (K, V)
static_assert(SMEM_BYTES <= 227 * 1024, "tiles do not fit shared memory");

__device__ __forceinline__ uint32_t tile_addr(uint32_t base, int row, int chunk) {
    return base + row * ROW_BYTES + ((chunk ^ (row & SWZ_MASK)) << 4);
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
    const int n = pred ? 16 : 0;      // n = 0 writes zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// `rows` rows x HD of bf16 from global rows (row stride `stride` elements) into a swizzled tile;
// rows >= n_valid are filled with zeros.
__device__ __forceinline__ void load_tile(uint32_t smem, const bf16* src, size_t stride, int rows, int n_valid) {
    for (int idx = threadIdx.x; idx < rows * CHUNKS; idx += THREADS) {
        const int row = idx / CHUNKS, chunk = idx % CHUNKS;
        const bool ok = row < n_valid;
        cp_async16(tile_addr(smem, row, chunk), src + (size_t)(ok ? row : 0) * stride + chunk * 8, ok);
    }
}

// A tile of keys (or values) whose rows before position `start` come from the cache line and the others from
// the step's buffer; rows >= n_valid are filled with zeros.  `src` points at the row that position k0 would have.
__device__ __forceinline__ void load_tile_mixed(uint32_t smem, const bf16* src, size_t stride, int rows, int n_valid, int k0,
                                                int start, const CachedPrefix& cached, const bf16* pool, int slot, int nkv,
                                                int kvh) {
    for (int idx = threadIdx.x; idx < rows * CHUNKS; idx += THREADS) {
        const int row = idx / CHUNKS, chunk = idx % CHUNKS;
        const bool ok = row < n_valid;
        const bf16* p = src + chunk * 8;
        if (ok) p = k0 + row < start ? pool + cached_row(cached, slot, k0 + row, nkv, kvh, HD) + chunk * 8
                                     : p + (size_t)row * stride;
        cp_async16(tile_addr(smem, row, chunk), p, ok);
    }
}

// EXT: sequences may go on from what earlier steps stored (`cached`); positions are then absolute, q0 and `len`
// count the step's own tokens of the sequence, and seq_len holds the lengths after the step.
template <bool EXT>
__global__ void __launch_bounds__(THREADS)
attn_prefill_mma_kernel(const bf16* __restrict__ q_src, const bf16* __restrict__ kv_src,
                        const int* __restrict__ seq_first_row, const int* __restrict__ seq_len, int n_seq,
                        bf16* __restrict__ out, int nq, int nkv, int q_row_heads, int kv_row_heads,
                        int kv_k_head0, float scale, float cap, int window, int parts, int piece,
                        float* __restrict__ partial, CachedPrefix cached) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    // Which sequence, which tile of BM queries and which part of its keys is this CTA's.  Items are handed
    // out from the end of the list: the last tiles of a sequence see the most keys and should start first.
    // (heads vary fastest in the grid, so the long items of all heads come before anyone's short ones).
    const int item = (int)gridDim.y - 1 - (int)blockIdx.y;
    const int gtile = item / parts, part = item % parts;
    int seq = -1, q0 = 0, len = 0;
    grid_dependents_launch();
    // (the step's tables were written before the step's first kernel: the tile is found before the wait)
    const bool found = find_tile(gtile, seq_len, n_seq, seq, q0, len, EXT ? cached.seq_start : nullptr);
    grid_dependency_wait();
    if (!found) return;
    const int head = blockIdx.x;
    const int kvh = head / (nq / nkv);
    const int first = seq_first_row[seq];             // row of the sequence's first token of this step
    const int start = EXT ? cached.seq_start[seq] : 0;         // its position
    const int slot = EXT ? cached.seq_slot[seq] : -1;
    const int total = start + len;                    // keys the sequence has after the step
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;

    const uint32_t sQ = (uint32_t)__cvta_generic_to_shared(smem_raw);
    const uint32_t sKV = sQ + Q_BYTES;                // stage s: K at sKV + s * 2 KV_BYTES, V right after

    const size_t q_stride = (size_t)q_row_heads * HD, kv_stride = (size_t)kv_row_heads * HD;
    int k_first, n_tiles;
    key_tiles(q0, len, window, k_first, n_tiles, start);
    const int np = pf::parts_of(n_tiles, parts, piece);
    const bool shared_tile = np > 1;
    if (part >= np) return;
    if (shared_tile) {                                               // this part's share of the key tiles
        const int t0 = (int)((long long)n_tiles * part / np), t1 = (int)((long long)n_tiles * (part + 1) / np);
        k_first += t0 * BN;
        n_tiles = t1 - t0;
    }
    // the row that position 0 would have in the step's buffer (before it when the sequence goes on: never read)
    const bf16* kbase = kv_src + ((ptrdiff_t)first - start) * (ptrdiff_t)kv_stride + (size_t)(kv_k_head0 + kvh) * HD;
    const bf16* vbase = kbase + (size_t)nkv * HD;
    auto load_kv = [&](int it) {
        const int k0 = k_first + it * BN;
        const uint32_t dst = sKV + (it & 1) * 2 * KV_BYTES;
        const int n_keys = min(BN, total - k0);
        if (EXT && k0 < start && slot >= 0) {
            load_tile_mixed(dst, kbase + (ptrdiff_t)k0 * (ptrdiff_t)kv_stride, kv_stride, BN, n_keys, k0, start, cached,
                            (const bf16*)cached.kpool, slot, nkv, kvh);
            load_tile_mixed(dst + KV_BYTES, vbase + (ptrdiff_t)k0 * (ptrdiff_t)kv_stride, kv_stride, BN, n_keys, k0, start,
                            cached, (const bf16*)cached.vpool, slot, nkv, kvh);
            return;
        }
        load_tile(dst, kbase + (ptrdiff_t)k0 * (ptrdiff_t)kv_stride, kv_stride, BN, n_keys);
        load_tile(dst + KV_BYTES, vbase + (ptrdiff_t)k0 * (ptrdiff_t)kv_stride, kv_stride, BN, n_keys);
    };
    load_tile(sQ, q_src + (size_t)(first + q0) * q_stride + (size_t)head * HD, q_stride, BM, min(BM, len - q0));
    load_kv(0);
    asm volatile("cp.async.commit_group;\n" ::: "memory");

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[i][c] = 0.f;
    // running maximum in units of log2(e): exp(s - m) = 2^(s log2e - m log2e)
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float LOG2E = 1.4426950408889634f;
    const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;
    const float cap2 = cap * LOG2E, scale2 = scale * LOG2E;

    const int row_lo = start + q0 + warp * 16 + g;    // this thread's two query positions
    const int row_hi = row_lo + 8;
    const int warp_first = start + q0 + warp * 16, warp_last = warp_first + 15;

    for (int it = 0; it < n_tiles; ++it) {
        const int k0 = k_first + it * BN;
        if (it + 1 < n_tiles) load_kv(it + 1);        // the other stage: its readers finished a tile ago
        asm volatile("cp.async.commit_group;\n" ::: "memory");
        asm volatile("cp.async.wait_group 1;\n" ::: "memory");     // this tile (and Q) has landed
        __syncthreads();
        const uint32_t sK = sKV + (it & 1) * 2 * KV_BYTES, sV = sK + KV_BYTES;

        // a warp whose rows see none of this tile's keys (all later, or all outside the window) skips it
        const bool any = k0 <= warp_last && (window <= 0 || k0 + BN - 1 > warp_first - window);
        if (any) {
            // S = Q K^T for this warp's 16 rows and the 64 keys of the tile
            float s[BN / 8][4];
#pragma unroll
            for (int j = 0; j < BN / 8; ++j)
#pragma unroll
                for (int c = 0; c < 4; ++c) s[j][c] = 0.f;
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
                uint32_t a[4];
                ldmatrix_x4(a, tile_addr(sQ, warp * 16 + (lane & 15), kk * 2 + (lane >> 4)));
#pragma unroll
                for (int jp = 0; jp < BN / 16; ++jp) {
                    uint32_t b[4];
                    ldmatrix_x4(b, tile_addr(sK, jp * 16 + (lane & 7) + ((lane >> 4) << 3), kk * 2 + ((lane >> 3) & 1)));
                    mma16816(s[2 * jp], a, b[0], b[1]);
                    mma16816(s[2 * jp + 1], a, b[2], b[3]);
                }
            }
            // scale, cap, mask; scores end up in units of log2(e)
            const bool inner = k0 + BN - 1 <= warp_first && k0 + BN <= total &&
                               (window <= 0 || k0 > warp_last - window);   // every key seen by every row
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < BN / 8; ++j)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    float v = cap > 0.f ? cap2 * fast_tanh(s[j][c] * scale * inv_cap) : s[j][c] * scale2;
                    if (!inner) {
                        const int key = k0 + j * 8 + t * 2 + (c & 1);
                        const int row = (c & 2) ? row_hi : row_lo;
                        const bool seen = key <= row && key < total && (window <= 0 || key > row - window);
                        v = seen ? v : -INFINITY;
                    }
                    s[j][c] = v;
                    mx[c >> 1] = fmaxf(mx[c >> 1], v);
                }
            float corr[2], m_use[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m_run[r], mx[r]);
                m_use[r] = m_new == -INFINITY ? 0.f : m_new;      // a row that has seen no key yet
                corr[r] = ex2(m_run[r] - m_use[r]);                // 2^(-inf) = 0
                m_run[r] = m_new;
                l_run[r] *= corr[r];
            }
            uint32_t p[BN / 16][4];
#pragma unroll
            for (int j = 0; j < BN / 8; ++j) {
                const float p0 = ex2(s[j][0] - m_use[0]), p1 = ex2(s[j][1] - m_use[0]);
                const float p2 = ex2(s[j][2] - m_use[1]), p3 = ex2(s[j][3] - m_use[1]);
                l_run[0] += p0 + p1;
                l_run[1] += p2 + p3;
                p[j >> 1][(j & 1) * 2] = pack_bf16(p0, p1);
                p[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
            }
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) {
                o[i][0] *= corr[0];
                o[i][1] *= corr[0];
                o[i][2] *= corr[1];
                o[i][3] *= corr[1];
            }
            // O += P V
#pragma unroll
            for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
                for (int ip = 0; ip < HD / 16; ++ip) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, tile_addr(sV, kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), ip * 2 + (lane >> 4)));
                    mma16816(o[2 * ip], p[kk], b[0], b[1]);
                    mma16816(o[2 * ip + 1], p[kk], b[2], b[3]);
                }
            }
        }
        __syncthreads();                              // this stage may be overwritten by the load after next
    }

    // the sums of a row are spread over the four threads that share it
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    if (shared_tile) {
        // maximum (in units of log2 e), sum and unnormalised output of this part; a row that saw no key: -inf, 0, 0
        float* base = partial + ((((size_t)gtile * nq + head) * parts + part) * BM) * PART_ROW;
        float* p_lo = base + (size_t)(warp * 16 + g) * PART_ROW;
        float* p_hi = p_lo + 8 * PART_ROW;
        if (t == 0) {
            p_lo[0] = m_run[0]; p_lo[1] = l_run[0];
            p_hi[0] = m_run[1]; p_hi[1] = l_run[1];
        }
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            *reinterpret_cast<float2*>(p_lo + 2 + i * 8 + t * 2) = make_float2(o[i][0], o[i][1]);
            *reinterpret_cast<float2*>(p_hi + 2 + i * 8 + t * 2) = make_float2(o[i][2], o[i][3]);
        }
        return;
    }
    const float inv_lo = 1.0f / l_run[0], inv_hi = 1.0f / l_run[1];
    bf16* out_lo = out + (size_t)(first + row_lo - start) * nq * HD + (size_t)head * HD + t * 2;
    bf16* out_hi = out + (size_t)(first + row_hi - start) * nq * HD + (size_t)head * HD + t * 2;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
        if (row_lo < total) *reinterpret_cast<uint32_t*>(out_lo + i * 8) = pack_bf16(o[i][0] * inv_lo, o[i][1] * inv_lo);
        if (row_hi < total) *reinterpret_cast<uint32_t*>(out_hi + i * 8) = pack_bf16(o[i][2] * inv_hi, o[i][3] * inv_hi);
    }
}

// Adds the parts of the shared tiles: out = sum_p o_p 2^(m_p - m) / sum_p l_p 2^(m_p - m), parts in index order.
// A thread has one piece of 4 outputs of a row and asks for all parts' maxima at once, then for all their sums
// and outputs at once: two round trips to the scratch (which the attention kernel has just written: L2), not
// two per part.
constexpr int MAX_PARTS = 4;
constexpr int MERGE_ROWS = 8;                         // rows of the tile per CTA

__global__ void __launch_bounds__(256)
attn_prefill_merge_kernel(const float* __restrict__ partial, const int* __restrict__ seq_first_row,
                          const int* __restrict__ seq_len, int n_seq, bf16* __restrict__ out, int nq, int window,
                          int parts, int piece, const int* __restrict__ seq_start) {
    const int gtile = blockIdx.x, head = blockIdx.y;
    const int r_begin = blockIdx.z * MERGE_ROWS;
    // the step's tables were written before the attention kernel started: they are read while it still runs
    int seq = -1, q0 = 0, len = 0;
    const bool found = find_tile(gtile, seq_len, n_seq, seq, q0, len, seq_start);
    int k_first = 0, n_tiles = 0;
    if (found) key_tiles(q0, len, window, k_first, n_tiles, seq_start ? seq_start[seq] : 0);
    const int np = found ? parts_of(n_tiles, parts, piece) : 1;
    const int first = found ? seq_first_row[seq] : 0;
    grid_dependents_launch();
    grid_dependency_wait();
    if (np <= 1) return;
    const int rows = min(MERGE_ROWS, len - q0 - r_begin);
    const float* base = partial + (((size_t)gtile * nq + head) * parts * BM) * PART_ROW;
    constexpr int VEC = HD / 4;                       // pieces of 4 outputs in a row
    for (int idx = threadIdx.x; idx < rows * VEC; idx += blockDim.x) {
        const int r = r_begin + idx / VEC, c = (idx % VEC) * 4;
        const float* row0 = base + (size_t)r * PART_ROW;
        float mp[MAX_PARTS];
        float m = -INFINITY;
#pragma unroll
        for (int p = 0; p < MAX_PARTS; ++p) {
            mp[p] = p < np ? row0[(size_t)p * BM * PART_ROW] : -INFINITY;
            m = fmaxf(m, mp[p]);
        }
        float lp[MAX_PARTS];
        float2 a[MAX_PARTS], b[MAX_PARTS];
#pragma unroll
        for (int p = 0; p < MAX_PARTS; ++p) {
            const float* row = row0 + (size_t)p * BM * PART_ROW;
            const bool has = p < np;
            lp[p] = has ? row[1] : 0.f;
            a[p] = has ? *reinterpret_cast<const float2*>(row + 2 + c) : make_float2(0.f, 0.f);
            b[p] = has ? *reinterpret_cast<const float2*>(row + 4 + c) : make_float2(0.f, 0.f);
        }
        float l = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int p = 0; p < MAX_PARTS; ++p) {
            if (mp[p] == -INFINITY) continue;         // no such part, or it saw no key of the row
            const float w = ex2(mp[p] - m);
            l += lp[p] * w;
            acc[0] += a[p].x * w; acc[1] += a[p].y * w; acc[2] += b[p].x * w; acc[3] += b[p].y * w;
        }
        const float inv = 1.0f / l;
        bf16* o = out + (size_t)(first + q0 + r) * nq * HD + (size_t)head * HD + c;
        *reinterpret_cast<uint2*>(o) = make_uint2(pack_bf16(acc[0] * inv, acc[1] * inv), pack_bf16(acc[2] * inv, acc[3] * inv));
    }
}

}  // namespace pf
}  // namespace janis

using namespace janis;

JANIS_EXPORT int janis_attn_prefill_tile() { return pf::BM; }

static int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
    }
    return n;
}

// The most CTAs that share a tile of queries in a step of n_tiles_bound tiles and nq heads (1: none is shared),
// and the floats of scratch such a step needs (0 when nothing is shared).
JANIS_EXPORT int janis_attn_prefill_parts(int n_tiles_bound, int nq) {
    return (long long)n_tiles_bound * nq < 2LL * sm_count() ? pf::MAX_PARTS : 1;
}
JANIS_EXPORT long long janis_attn_prefill_scratch(int n_tiles_bound, int nq) {
    const int parts = janis_attn_prefill_parts(n_tiles_bound, nq);
    return parts > 1 ? (long long)n_tiles_bound * nq * parts * pf::BM * pf::PART_ROW : 0;
}

static int g_prefill_piece = 0;     // key tiles per piece of a shared tile of queries; 0: chosen from the step's size

// Fixes the size of the pieces that shared tiles of queries are cut into (0: automatic again).
JANIS_EXPORT void janis_attn_set_prefill_piece(int piece) { g_prefill_piece = piece > 0 ? piece : 0; }

// How long a step takes whose shared tiles are cut into pieces of `piece` key tiles, in microseconds, by a model
// of five numbers fitted to a B200 at head size 256 (60 timings of 1 to 7 prompts of 300 to 4,096 tokens and
// pieces of 4 to "nothing shared", 5 % off on average): a CTA's item costs `cta` besides its tiles (7.1 us for the
// tcgen05 kernel: Q and the first keys, the tiles the softmax runs behind, the masked tiles at the diagonal, the way
// out; 9.9 us before P moved to tensor memory), `tile` per key tile (1.22 us), 1.8 us more when it leaves a partial
// result, and a step with shared tiles 6 us for the places of parts that come to nothing and for the merge's
// launch, plus 0.45 us per round of partial rows.  CTAs go to the SM that is free first, in the order of their
// launch.  The step's lengths are on the device: the model takes n_seq sequences of equal length.
static double prefill_model_us(int n_seq, int len, int nq, int window, int parts, int piece, int sms, double cta,
                               double tile, int* longest) {
    std::vector<std::pair<int, bool>> items;          // key tiles, leaves a partial result; in tile order
    long long split_parts = 0;
    *longest = 0;
    for (int q0 = 0; q0 < len; q0 += pf::BM) {
        int k_first, n;
        pf::key_tiles(q0, len, window, k_first, n);
        *longest = std::max(*longest, n);
        const int np = pf::parts_of(n, parts, piece);
        for (int p = 0; p < np; ++p) items.push_back({(int)((long long)n * (p + 1) / np - (long long)n * p / np), np > 1});
        if (np > 1) split_parts += np;
    }
    std::priority_queue<double, std::vector<double>, std::greater<double>> free_at;
    for (int i = 0; i < sms; ++i) free_at.push(0.0);
    double end = 0.0;
    for (int s = n_seq - 1; s >= 0; --s)              // the last tile of the last sequence is launched first
        for (int i = (int)items.size() - 1; i >= 0; --i)
            for (int h = 0; h < nq; ++h) {
                const double t = free_at.top() + cta + tile * items[i].first + (items[i].second ? 1.8 : 0.0);
                free_at.pop();
                free_at.push(t);
                end = std::max(end, t);
            }
    if (split_parts) end += 6.0 + 0.45 * (double)(split_parts * n_seq * nq) / sms;
    return end;
}

// The piece that the model likes best for a step (the largest among equals: fewer partial results), remembered per
// shape of step with the lengths rounded up to whole tiles of queries, so that few shapes are ever asked about.  The
// candidates are multiples of an SM's even share of the key tiles (the best lay between 1.25 and 2 of it wherever it
// was measured), a few small pieces, and "nothing shared": a piece as long as the longest tile's keys.
static int prefill_piece_for(int n_tok, int n_seq, int nq, int window, int parts, bool tc05, int* longest) {
    static std::map<std::tuple<int, int, int, int, int, bool>, std::pair<int, int>> known;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    const int len = ((n_tok + n_seq - 1) / n_seq + pf::BM - 1) / pf::BM * pf::BM;
    const auto key = std::make_tuple(len, n_seq, nq, window > 0 && window < len ? window : 0, parts, tc05);
    auto it = known.find(key);
    if (it == known.end()) {
        const int sms = sm_count();
        // per key tile: the softmax's share does not depend on the head size, the products' does; the mma.sync
        // kernel took 2.7 times as long per tile at head size 256 and has less to do around its tiles
        const double tile = tc05 ? 1.0 + 0.22 * pf::HD / 256.0 : 3.9 * pf::HD / 256.0, cta = tc05 ? 7.1 : 6.0;
        int most = 0, best = 4;
        double best_us = prefill_model_us(n_seq, len, nq, window, parts, 4, sms, cta, tile, &most);
        long long key_tiles = 0;
        for (int q0 = 0; q0 < len; q0 += pf::BM) {
            int k_first, n;
            pf::key_tiles(q0, len, window, k_first, n);
            key_tiles += n;
        }
        const double share = (double)key_tiles * n_seq * nq / sms;
        std::vector<int> tries = {5, 6, 8};
        for (double m : {1.0, 1.25, 1.5, 1.75, 2.0, 2.5, 3.0}) tries.push_back((int)(m * share + 0.5));
        std::sort(tries.begin(), tries.end());
        for (int piece : tries) {
            if (piece <= 4 || piece >= most) continue;
            int unused;
            const double us = prefill_model_us(n_seq, len, nq, window, parts, piece, sms, cta, tile, &unused);
            if (us <= best_us) { best_us = us; best = piece; }
        }
        if (most > 4) {                                // and nothing shared at all
            int unused;
            if (prefill_model_us(n_seq, len, nq, window, 1, most, sms, cta, tile, &unused) <= best_us) best = most;
        }
        if (known.size() > 4096) known.clear();
        it = known.emplace(key, std::make_pair(best, most)).first;
    }
    *longest = it->second.second;
    return it->second.first;
}

// What the step of these sizes would be cut into (for tests and measurements): the piece, in key tiles.
JANIS_EXPORT int janis_attn_prefill_piece(int n_tok, int n_seq, int n_tiles_bound, int nq, int window, int tc05) {
    if (n_seq <= 0 || n_tok <= 0) return 0;
    int longest = 0;
    return prefill_piece_for(n_tok, n_seq, nq, window, janis_attn_prefill_parts(n_tiles_bound, nq), tc05 != 0, &longest);
}

static int g_prefill_kernels = 0;   // kernels that the last call of janis_attn_prefill_mma launched
JANIS_EXPORT int janis_attn_prefill_kernels() { return g_prefill_kernels; }

static int g_prefill_kernel = 1;    // 1: tcgen05 where the head size allows it, else mma.sync; 0: mma.sync always

// Which kernel janis_attn_prefill_mma launches (both give the same results up to rounding).
JANIS_EXPORT void janis_attn_set_prefill_kernel(int which) { g_prefill_kernel = which ? 1 : 0; }

// q_src: [n_tok, q_row_heads, hd] with the queries in its first nq heads; keys and values of position j of
// sequence s are read from row seq_first_row[s] + j of kv_src [n_tok, kv_row_heads, hd], key heads starting at
// head kv_k_head0, value heads nkv later.  n_tiles_bound >= sum over sequences of ceil(len / tile), tile =
// janis_attn_prefill_tile().  partial: janis_attn_prefill_scratch(n_tiles_bound, nq) floats, or null (or
// fewer floats), in which case no tile is shared.
// With seq_start (int32 [n_seq], tokens of each sequence that earlier steps stored) the step continues sequences:
// seq_len then holds the lengths after the step, seq_first_row the row of a sequence's first token of this step, and
// keys and values of positions below seq_start come from the cache line (kpool, vpool, page_table, ring_len as in
// janis_attn_decode); such a step runs on the mma.sync kernel.
JANIS_EXPORT int janis_attn_prefill_mma(const void* q_src, const void* kv_src, int n_tok, const int* seq_first_row,
                                        const int* seq_len, int n_seq, int n_tiles_bound, void* out, int nq,
                                        int nkv, int q_row_heads, int kv_row_heads, int kv_k_head0, float scale,
                                        float cap, int window, float* partial, long long partial_floats,
                                        const int* seq_start, const int* seq_slot, const void* kpool, const void* vpool,
                                        const int* page_table, int table_stride, int ring_len, int max_len,
                                        cudaStream_t stream) {
    if (n_seq <= 0 || n_tiles_bound <= 0) return 0;
    if (nkv <= 0 || nq % nkv) return fail("attn_prefill_mma: %d query heads do not divide over %d key heads", nq, nkv);
    if (((uintptr_t)q_src | (uintptr_t)kv_src | (uintptr_t)out | (uintptr_t)partial | (uintptr_t)kpool | (uintptr_t)vpool) & 15)
        return fail("attn_prefill_mma: operands must be 16-byte aligned");
    const bool ext = seq_start != nullptr;
    if (ext && (seq_slot == nullptr || kpool == nullptr || vpool == nullptr || page_table == nullptr))
        return fail("attn_prefill_mma: sequences that continue need their slots and the cache line");
    if (ring_len % JANIS_PAGE) return fail("attn_prefill_mma: ring length %d is not a multiple of the page", ring_len);
    const CachedPrefix cached = {seq_start, seq_slot, kpool, vpool, page_table, table_stride, ring_len};
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(pf::attn_prefill_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             pf::SMEM_BYTES);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(pf::attn_prefill_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     pf::SMEM_BYTES);
        if (e != cudaSuccess) return fail("attn_prefill_mma: shared memory of %d bytes refused: %s", pf::SMEM_BYTES,
                                          cudaGetErrorString(e));
        configured = true;
    }
    int parts = janis_attn_prefill_parts(n_tiles_bound, nq);
    if (partial == nullptr || partial_floats < janis_attn_prefill_scratch(n_tiles_bound, nq)) parts = 1;
    // The pieces that shared tiles of queries are cut into: what a model of the step's time likes best.  When that
    // is "none shared", the step is launched without the places of the parts and without the merge.
    const bool tc05 = g_prefill_kernel == 1 && !ext && pf::TC05_HEAD;
    int piece = g_prefill_piece;
    if (piece <= 0 && parts > 1) {
        int longest = 0;
        piece = prefill_piece_for(n_tok, n_seq, nq, window, parts, tc05, &longest);
    }
    if (piece <= 0) piece = 4;
    // No tile of queries has more key tiles than the step's longest sequence has (when the sequences start with the
    // step): places for parts that no tile can have would be CTAs that only come and go (2 to 3 us each for a CTA of
    // this size), and a piece that no tile exceeds means that nothing is shared: no places for parts, no merge.
    // (max_len: the longest sequence's tokens in this step, when the host knows them; else the step's tokens bound it)
    int most_tiles = ((max_len > 0 ? std::min(max_len, n_tok) : n_tok) + pf::BN - 1) / pf::BN;
    if (window > 0) most_tiles = std::min(most_tiles, (window + pf::BM) / pf::BN + 1);        // a window bounds a tile's keys
    if (!ext && parts > 1) parts = std::max(1, std::min(parts, (most_tiles + piece - 1) / piece));
    if (!ext && most_tiles <= 8) parts = 1;           // up to 512 keys a tile: sharing measured no faster (512 tokens: 17.0 against 16.5 us)
    if ((long long)n_tiles_bound * parts > 65535) return fail("attn_prefill_mma: %d tiles of queries exceed the grid", n_tiles_bound);
    int done = -1;
    if (g_prefill_kernel == 1 && !ext)                // the tcgen05 kernel takes sequences that start at position 0
        done = launch_prefill_tc05(q_src, kv_src, n_tok, seq_first_row, seq_len, n_seq, n_tiles_bound, out, nq, nkv,
                                   q_row_heads, kv_row_heads, kv_k_head0, scale, cap, window, parts, piece, partial,
                                   stream);
    if (done > 0) return 1;
    if (done < 0) {
        dim3 grid(nq, n_tiles_bound * parts);
        auto kernel = ext ? pf::attn_prefill_mma_kernel<true> : pf::attn_prefill_mma_kernel<false>;
        if (launch_kernel("attn_prefill_mma", kernel, grid, dim3(pf::THREADS), pf::SMEM_BYTES, stream, 1, (const bf16*)q_src,
                          (const bf16*)kv_src, seq_first_row, seq_len, n_seq, (bf16*)out, nq, nkv, q_row_heads,
                          kv_row_heads, kv_k_head0, scale, cap, window, parts, piece, partial, cached))
            return 1;
    }
    g_prefill_kernels = parts == 1 ? 1 : 2;
    if (parts == 1) return 0;
    return launch_kernel("attn_prefill_merge", pf::attn_prefill_merge_kernel, dim3(n_tiles_bound, nq, pf::BM / pf::MERGE_ROWS), dim3(256), 0, stream, 1,
                         (const float*)partial, seq_first_row, seq_len, n_seq, (bf16*)out, nq, window, parts, piece,
                         seq_start);
}
