// What the two prompt-attention kernels of a head size share: the tile sizes, how a CTA finds its tile of
// queries and the key tiles it walks, the layout of the partial results of shared tiles, and the fast
// exponential and tanh.
#pragma once

#include "common.cuh"

#ifndef JANIS_HEAD_DIM
#error "compile with -DJANIS_HEAD_DIM=<head size, a multiple of 16>"
#endif

namespace janis {
namespace pf {

constexpr int HD = JANIS_HEAD_DIM;
constexpr int BN = HD <= 256 ? 64 : 32;               // keys per tile
constexpr int WARPS = HD <= 256 ? 8 : 4;              // 16 query rows each (mma.sync kernel)
constexpr int BM = WARPS * 16;                        // queries per tile
constexpr int PART_ROW = HD + 2;                      // floats of a partial row: maximum, sum, output
constexpr bool TC05_HEAD = HD % 64 == 0 && HD <= 256; // head sizes that the tcgen05 kernel takes

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float ex2(float x) {        // 2^x; ex2(-inf) = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float fast_tanh(float x) {  // 1 - 2 / (e^2x + 1); exact limits at +-inf
    const float e = ex2(x * 2.8853900817779268f);      // 2 log2(e)
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;\n" : "=f"(r) : "f"(e + 1.0f));
    return 1.0f - 2.0f * r;
}

// The sequence and the tile of BM queries that item `tile` of the step stands for (false: none).  `len` is the
// number of tokens the sequence brings to this step: seq_end[s], less what earlier steps stored (seq_start[s],
// when the step continues sequences), and q0 counts from the first of them.
__device__ __forceinline__ bool find_tile(int tile, const int* __restrict__ seq_end, int n_seq, int& seq, int& q0, int& len,
                                          const int* __restrict__ seq_start = nullptr) {
    for (int s = 0; s < n_seq; ++s) {
        const int n = seq_end[s] - (seq_start ? seq_start[s] : 0);
        const int nt = (n + BM - 1) / BM;
        if (tile < nt) { seq = s; q0 = tile * BM; len = n; return true; }
        tile -= nt;
    }
    return false;
}

// Key tiles [k_first / BN, ...) that a tile of queries walks: n_tiles of them from key k_first (an absolute
// position; the step's first token stands at position `start`).
__host__ __device__ __forceinline__ void key_tiles(int q0, int len, int window, int& k_first, int& n_tiles, int start = 0) {
    const int q_last = start + min(q0 + BM, len) - 1;
    const int j_first = window > 0 ? max(0, start + q0 - window + 1) : 0;
    k_first = (j_first / BN) * BN;
    n_tiles = (q_last - k_first) / BN + 1;
}

// CTAs that share a tile of queries with n_tiles key tiles: pieces of at most `piece` key tiles, but no more
// than `parts` of them (1: the tile is one CTA's, which writes the output itself).  The attention kernels and
// the merge kernel decide the same way.
__host__ __device__ __forceinline__ int parts_of(int n_tiles, int parts, int piece) {
    const int want = (n_tiles + piece - 1) / piece;
    return parts <= 1 || want <= 1 ? 1 : (want < parts ? want : parts);
}

}  // namespace pf

// The tcgen05 kernel of the same step (attention_prefill_tc05.cu): 0 launched, 1 failed (message set),
// -1 this head size or these operands are not for it.
int launch_prefill_tc05(const void* q_src, const void* kv_src, int n_tok, const int* seq_first_row, const int* seq_len,
                        int n_seq, int n_tiles_bound, void* out, int nq, int nkv, int q_row_heads, int kv_row_heads,
                        int kv_k_head0, float scale, float cap, int window, int parts, int piece, float* partial,
                        cudaStream_t stream);

}  // namespace janis
