// Row-wise kernels of the residual stream: embedding gather, RMS norms (alone,
// and fused with the residual sum and the next norm), the gated activation,
// and the rotary encoding fused with the write of keys and values into the
// paged cache.  Sums of squares, reciprocal roots, angles and the residual sum
// are float; storage types only decide what is read and written.
#include "common.cuh"

namespace janis {

// ---------------------------------------------------------------------------
// embedding: out[t, :] = float(table[tokens[t], :]) * scale        (float rows)
// ---------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                             float* __restrict__ out, int H, int V, float scale) {
    const int t = blockIdx.x;
    grid_dependents_launch();
    grid_dependency_wait();                 // the tokens may come from the sampling kernel of the step before
    int tok = tokens[t];
    if (tok < 0 || tok >= V) tok = 0;   // the host has checked the ids; padding rows carry 0
    const T* row = table + (size_t)tok * H;
    float* o = out + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_float(row[i]) * scale;
}

// ---------------------------------------------------------------------------
// y[r, :] = x[src(r), :] * rsqrt(mean(x^2) + eps) * w      (w already holds offset + weight)
// ---------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void rmsnorm_kernel(const TI* __restrict__ x, const float* __restrict__ w,
                               const int* __restrict__ rows, TO* __restrict__ y, int H, float eps) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    grid_dependents_launch();
    grid_dependency_wait();
    const int src = rows ? rows[r] : r;
    const TI* xr = x + (size_t)src * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = to_float(xr[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    TO* yr = y + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) yr[i] = from_float<TO>(to_float(xr[i]) * inv * w[i]);
}

// ---------------------------------------------------------------------------
// h[r, :] += norm(res[r, :]; w_post)           (the residual sum, float, in place;
//                                               res itself when there is no w_post)
// y[r, :]  = norm(h[r, :]; w_next)             (only when w_next is given)
// `res` may be the sum of `n_part` partial results laid out [n_part, rows, H].
// ---------------------------------------------------------------------------
template <typename TR, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const TR* __restrict__ res, int n_part,
                                   size_t part_stride, const float* __restrict__ w_post, float eps_post,
                                   const float* __restrict__ w_next, float eps_next,
                                   TO* __restrict__ y, int H) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const TR* rr = res + (size_t)r * H;
    float* hr = h + (size_t)r * H;
    grid_dependents_launch();
    grid_dependency_wait();
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = to_float(rr[i]);
        for (int p = 1; p < n_part; ++p) v += to_float(rr[p * part_stride + i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    // without a post norm (w_post == nullptr) the result is added as it is
    const float inv = w_post ? 1.0f / sqrtf(ss / (float)H + eps_post) : 1.0f;
    float ss2 = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = to_float(rr[i]);
        for (int p = 1; p < n_part; ++p) v += to_float(rr[p * part_stride + i]);
        const float hv = hr[i] + (w_post ? v * inv * w_post[i] : v);
        hr[i] = hv;                         // read back below by this same thread only
        ss2 = fmaf(hv, hv, ss2);
    }
    if (w_next == nullptr) return;
    ss2 = block_sum(ss2, scratch);
    const float inv2 = 1.0f / sqrtf(ss2 / (float)H + eps_next);
    TO* yr = y + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) yr[i] = from_float<TO>(hr[i] * inv2 * w_next[i]);
}

// 8 consecutive elements as floats (p aligned to 16 bytes)
__device__ __forceinline__ void load8(const bf16* p, float* o) { Vec16<bf16>::load(p, o); }
__device__ __forceinline__ void load8(const float* p, float* o) {
    Vec16<float>::load(p, o);
    Vec16<float>::load(p + 4, o + 4);
}
__device__ __forceinline__ void store8(bf16* p, const float* v) { Vec16<bf16>::store(p, v); }
__device__ __forceinline__ void store8(float* p, const float* v) {
    Vec16<float>::store(p, v);
    Vec16<float>::store(p + 4, v + 4);
}

// The same with the row held in registers: NT threads take the row as vectors of 8 elements
// (H a multiple of 8, H <= 8 NT VPT) and every input is read once with 16-byte loads.  HOIST: the
// norms' weights are asked for together with the row (few rows, decoding: one round of latency
// less); otherwise they are read when they are needed, which leaves registers for more rows an SM.
template <typename TR, typename TO, int VPT, int NT, bool HOIST>
__global__ void __launch_bounds__(NT)
add_rmsnorm_vec_kernel(float* __restrict__ h, const TR* __restrict__ res, int n_part, size_t part_stride,
                       const float* __restrict__ w_post, float eps_post, const float* __restrict__ w_next,
                       float eps_next, TO* __restrict__ y, int H) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int nvec = H >> 3;
    const TR* rr = res + (size_t)r * H;
    float* hr = h + (size_t)r * H;
    float v[VPT][8], hv[VPT][8], wp[HOIST ? VPT : 1][8], wn[HOIST ? VPT : 1][8];
    grid_dependents_launch();
    grid_dependency_wait();
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int j = threadIdx.x + k * NT;
        if (j < nvec) {
            load8(rr + j * 8, v[k]);
            for (int p = 1; p < n_part; ++p) {
                float more[8];
                load8(rr + p * part_stride + j * 8, more);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[k][e] += more[e];
            }
            load8(hr + j * 8, hv[k]);
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[k][e] = 0.f;
        }
    }
    if (HOIST) {
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            const int j = threadIdx.x + k * NT;
            if (j < nvec) {
                if (w_post) load8(w_post + j * 8, wp[HOIST ? k : 0]);
                if (w_next) load8(w_next + j * 8, wn[HOIST ? k : 0]);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < VPT; ++k)
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(v[k][e], v[k][e], ss);
    ss = block_sum(ss, scratch);
    const float inv = w_post ? 1.0f / sqrtf(ss / (float)H + eps_post) : 1.0f;
    float ss2 = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int j = threadIdx.x + k * NT;
        if (j < nvec) {
            if (w_post) {
                float w[8];
                if (!HOIST) load8(w_post + j * 8, w);
#pragma unroll
                for (int e = 0; e < 8; ++e) hv[k][e] += v[k][e] * inv * (HOIST ? wp[HOIST ? k : 0][e] : w[e]);
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) hv[k][e] += v[k][e];
            }
            store8(hr + j * 8, hv[k]);
#pragma unroll
            for (int e = 0; e < 8; ++e) ss2 = fmaf(hv[k][e], hv[k][e], ss2);
        }
    }
    if (w_next == nullptr) return;
    ss2 = block_sum(ss2, scratch);
    const float inv2 = 1.0f / sqrtf(ss2 / (float)H + eps_next);
    TO* yr = y + (size_t)r * H;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int j = threadIdx.x + k * NT;
        if (j < nvec) {
            float w[8], o[8];
            if (!HOIST) load8(w_next + j * 8, w);
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = hv[k][e] * inv2 * (HOIST ? wn[HOIST ? k : 0][e] : w[e]);
            store8(yr + j * 8, o);
        }
    }
}

// ---------------------------------------------------------------------------
// gated activation over a fused [rows, 2*I] product whose columns alternate in
// groups of `group`: group g of gate columns, then group g of up columns.
// act: 0 = gelu (tanh form), 1 = silu
// ---------------------------------------------------------------------------
template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ gu, T* __restrict__ out, int rows, int I, int group,
                                 int act) {
    grid_dependents_launch();
    grid_dependency_wait();
    const size_t n = (size_t)rows * I;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int r = (int)(idx / I), j = (int)(idx % I);
        const size_t base = (size_t)r * 2 * I + (size_t)(j / group) * 2 * group + (j % group);
        const float g = to_float(gu[base]), u = to_float(gu[base + group]);
        const float a = act == 0 ? gelu_tanh(g) : g / (1.0f + expf(-g));
        out[idx] = from_float<T>(a * u);
    }
}

// The same for bfloat16 and groups of 8: a thread takes 8 gates and their 8 ups as two 16-byte loads.  With
// tanhf and expf the kernel was bound by instructions, not by memory (some forty a value, 19 million values a
// layer of a 2,048-token prompt); here tanh(x) = 1 - 2 / (e^2x + 1) and the sigmoid are built on ex2.approx and
// rcp.approx (absolute error near 2e-7, exact limits at +-inf), far below the rounding to bfloat16 that follows.
__device__ __forceinline__ float ex2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_fast(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float gelu_tanh_fast(float v) {
    const float inner = 0.7978845608028654f * (v + 0.044715f * v * v * v);
    const float t = 1.0f - 2.0f * rcp_fast(ex2_fast(inner * 2.8853900817779268f) + 1.0f);     // 2 log2(e)
    return 0.5f * v * (1.0f + t);
}
__device__ __forceinline__ float silu_fast(float v) {
    return v * rcp_fast(1.0f + ex2_fast(-v * 1.4426950408889634f));
}

template <int ACT>
__global__ void __launch_bounds__(256)
gated_act8_bf16_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, size_t n_groups) {
    grid_dependents_launch();
    grid_dependency_wait();
    for (size_t q = (size_t)blockIdx.x * blockDim.x + threadIdx.x; q < n_groups; q += (size_t)gridDim.x * blockDim.x) {
        float g[8], u[8], o[8];
        Vec16<bf16>::load(gu + q * 16, g);
        Vec16<bf16>::load(gu + q * 16 + 8, u);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = (ACT == 0 ? gelu_tanh_fast(g[e]) : silu_fast(g[e])) * u[e];
        Vec16<bf16>::store(out + q * 8, o);
    }
}

// ---------------------------------------------------------------------------
// x = cap * tanh(x / cap) in place over float values (the cap on logits that a library product made)
// ---------------------------------------------------------------------------
__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap) {
    const float inv = 1.0f / cap;
    grid_dependents_launch();
    grid_dependency_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] * inv);
}

// ---------------------------------------------------------------------------
// rotary encoding of q and k in place, and the write of k (rotated) and v into
// the paged cache.  qkv: [T, row_heads, hd], heads q, then k, then v (a layer that
// only reads another's keys has rows of q alone).  Pair (i, i + rot/2), i < rot/2;
// features from `rot` on pass through.  theta = float(pos) * inv_freq[i].
// A token of a sequence with slot < 0 (padding) is rotated but not stored.  With
// a ring (ring_len > 0) position p lives at p % ring_len and only positions
// >= seq_end - ring_len are stored, so that no two tokens of a step share a place.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void rope_store_kernel(T* __restrict__ qkv, const int* __restrict__ tok_pos,
                                  const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                                  const int* __restrict__ seq_end, const float* __restrict__ inv_freq,
                                  int rot, int nq, int nkv, int hd, int row_heads, T* __restrict__ kpool,
                                  T* __restrict__ vpool, const int* __restrict__ page_table,
                                  int table_stride, int ring_len, int n_heads, int heads_per_cta) {
    // A CTA takes heads [blockIdx.y * heads_per_cta, ...) of token blockIdx.x: heads 0..nq-1 are queries,
    // then nkv key heads, then nkv value heads (n_heads = nq when only queries are rotated).  Few tokens
    // (decoding) spread their heads over CTAs; many tokens take all heads of a token in one CTA.
    const int t = blockIdx.x;
    const int half = rot >> 1;
    grid_dependents_launch();
    // The step's tables (positions, slots, ends, pages) are written before the step's first kernel and
    // inv_freq is a constant of the model: the place in the cache and the angle are found before the wait.
    const int pos = tok_pos[t];
    long long place = -1;                    // element offset of this token's row of head 0 in a pool
    if (kpool != nullptr && n_heads > nq) {
        const int seq = tok_seq[t];
        const int slot = seq_slot[seq];
        int idx = pos;
        bool keep = slot >= 0;
        if (keep && ring_len > 0) {
            keep = pos >= seq_end[seq] - ring_len;
            idx = pos % ring_len;
        }
        if (keep) {
            const int page = page_table[(size_t)slot * table_stride + idx / JANIS_PAGE];
            place = ((long long)page * nkv * JANIS_PAGE + idx % JANIS_PAGE) * hd;
        }
    }
    // thread i owns the pair (i, i + half) below half and the single feature i from rot on
    const int i0 = threadIdx.x;
    float s0 = 0.f, c0 = 1.f;
    if (i0 < half) sincosf((float)pos * inv_freq[i0], &s0, &c0);
    grid_dependency_wait();
    const int h_end = min(n_heads, ((int)blockIdx.y + 1) * heads_per_cta);
    for (int head = blockIdx.y * heads_per_cta; head < h_end; ++head) {
        const bool is_k = head >= nq && head < nq + nkv, is_v = head >= nq + nkv;
        T* p = qkv + ((size_t)t * row_heads + head) * hd;
        T* dst = nullptr;                    // this head's row in the cache, if it is stored
        if (place >= 0 && (is_k || is_v))
            dst = (is_k ? kpool : vpool) + place + (size_t)(is_k ? head - nq : head - nq - nkv) * JANIS_PAGE * hd;
        if (is_v) {
            if (dst)
                for (int d = i0; d < hd; d += blockDim.x) dst[d] = p[d];
            continue;
        }
        for (int i = i0; i < hd; i += blockDim.x) {
            if (i < half) {
                float s = s0, c = c0;
                if (i != i0) sincosf((float)pos * inv_freq[i], &s, &c);
                const float a = to_float(p[i]), b = to_float(p[i + half]);
                float lo_f, hi_f;
                rotate_pair(a, b, s, c, lo_f, hi_f);
                const T lo = from_float<T>(lo_f), hi = from_float<T>(hi_f);
                p[i] = lo;
                p[i + half] = hi;
                if (dst) { dst[i] = lo; dst[i + half] = hi; }
            } else if (i >= rot) {
                if (dst) dst[i] = p[i];
            }
        }
    }
}

// The same for rot == hd with 16-byte accesses: a thread takes 8 neighbouring pairs (i, i + hd/2) of one
// token and walks over `heads_per_thread` heads with the same 8 angles.
template <typename T>
__global__ void __launch_bounds__(128)
rope_store_vec_kernel(T* __restrict__ qkv, const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                      const int* __restrict__ seq_slot, const int* __restrict__ seq_end,
                      const float* __restrict__ inv_freq, int n_tok, int nq, int nkv, int hd, int row_heads,
                      T* __restrict__ kpool, T* __restrict__ vpool, const int* __restrict__ page_table,
                      int table_stride, int ring_len, int n_heads, int heads_per_thread) {
    const int half = hd >> 1, vph = half >> 3;               // vectors of 8 pairs per head
    const int groups = (n_heads + heads_per_thread - 1) / heads_per_thread;
    const long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const bool live = u < (long long)n_tok * groups * vph;
    grid_dependents_launch();
    // tables of the step and constants of the model only, before the wait
    int t = 0, hg = 0, vi = 0, pos = 0;
    long long place = -1;
    float sn[8], cs[8];
    if (live) {
        vi = (int)(u % vph);
        hg = (int)((u / vph) % groups);
        t = (int)(u / ((long long)vph * groups));
        pos = tok_pos[t];
        if (kpool != nullptr && n_heads > nq) {
            const int seq = tok_seq[t];
            const int slot = seq_slot[seq];
            int idx = pos;
            bool keep = slot >= 0;
            if (keep && ring_len > 0) {
                keep = pos >= seq_end[seq] - ring_len;
                idx = pos % ring_len;
            }
            if (keep) {
                const int page = page_table[(size_t)slot * table_stride + idx / JANIS_PAGE];
                place = ((long long)page * nkv * JANIS_PAGE + idx % JANIS_PAGE) * hd;
            }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) sincosf((float)pos * inv_freq[vi * 8 + e], &sn[e], &cs[e]);
    }
    grid_dependency_wait();
    if (!live) return;
    const int h_end = min(n_heads, (hg + 1) * heads_per_thread);
    for (int head = hg * heads_per_thread; head < h_end; ++head) {
        const bool is_k = head >= nq && head < nq + nkv, is_v = head >= nq + nkv;
        T* p = qkv + ((size_t)t * row_heads + head) * hd + vi * 8;
        T* dst = nullptr;
        if (place >= 0 && (is_k || is_v))
            dst = (is_k ? kpool : vpool) + place + (size_t)(is_k ? head - nq : head - nq - nkv) * JANIS_PAGE * hd + vi * 8;
        float lo[8], hi[8];
        load8(p, lo);
        load8(p + half, hi);
        if (!is_v) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float a = lo[e], b = hi[e];
                rotate_pair(a, b, sn[e], cs[e], lo[e], hi[e]);
            }
            store8(p, lo);
            store8(p + half, hi);
        }
        if (dst) {
            store8(dst, lo);                                  // rounds as the store into the row did
            store8(dst + half, hi);
        }
    }
}

// ---------------------------------------------------------------------------
// keys and values of a step's rows into the paged cache, as a kernel of its own: a step that continues
// sequences attends first (its windowed lines still need the places that the step's own tokens will take)
// and stores afterwards.  Same places and the same rule for rings as the encoding kernels above.  A thread
// copies 16 bytes; units are (token, key or value head, piece).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
kv_store_kernel(const T* __restrict__ qkv, const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                const int* __restrict__ seq_slot, const int* __restrict__ seq_end, int n_tok, int nq, int nkv, int hd,
                int row_heads, T* __restrict__ kpool, T* __restrict__ vpool, const int* __restrict__ page_table,
                int table_stride, int ring_len) {
    constexpr int VEC = Vec16<T>::N;
    const int ppr = hd / VEC;                                   // pieces per head row
    const long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    grid_dependents_launch();
    grid_dependency_wait();
    if (u >= (long long)n_tok * 2 * nkv * ppr) return;
    const int pc = (int)(u % ppr), head = (int)((u / ppr) % (2 * nkv)), t = (int)(u / ((long long)ppr * 2 * nkv));
    const int pos = tok_pos[t], seq = tok_seq[t], slot = seq_slot[seq];
    if (slot < 0) return;
    int idx = pos;
    if (ring_len > 0) {
        if (pos < seq_end[seq] - ring_len) return;              // a later token of this step takes its place
        idx = pos % ring_len;
    }
    const int page = page_table[(size_t)slot * table_stride + idx / JANIS_PAGE];
    const bool is_v = head >= nkv;
    T* dst = (is_v ? vpool : kpool) + (((size_t)page * nkv + (is_v ? head - nkv : head)) * JANIS_PAGE + idx % JANIS_PAGE) * hd;
    const T* src = qkv + ((size_t)t * row_heads + nq + head) * hd;
    *reinterpret_cast<uint4*>(dst + pc * VEC) = *reinterpret_cast<const uint4*>(src + pc * VEC);
}

}  // namespace janis

using namespace janis;

static inline int row_threads(int H) { return H >= 2048 ? 512 : (H >= 512 ? 256 : 128); }

// 0: launch every kernel of this library plainly; 1 (default): let a kernel's CTAs arrive while the one before it runs
JANIS_EXPORT void janis_set_overlap(int on) { overlap_launches() = on ? 1 : 0; }

JANIS_EXPORT int janis_embed(const int* tokens, const void* table, int table_dtype, float* out, int T, int H,
                             int V, float scale, cudaStream_t stream) {
    if (T <= 0) return 0;
    const dim3 grid(T), block(row_threads(H));
    if (table_dtype == JANIS_F32)
        return launch_kernel("embed", embed_kernel<float>, grid, block, 0, stream, 1, tokens, (const float*)table, out, H, V,
                             scale);
    if (table_dtype == JANIS_BF16)
        return launch_kernel("embed", embed_kernel<bf16>, grid, block, 0, stream, 1, tokens, (const bf16*)table, out, H, V,
                             scale);
    return fail("embed: unknown table dtype %d", table_dtype);
}

JANIS_EXPORT int janis_rmsnorm(const void* x, int x_dtype, const float* w, const int* rows, void* y, int y_dtype,
                               int R, int H, float eps, cudaStream_t stream) {
    if (R <= 0) return 0;
    const dim3 grid(R), block(row_threads(H));
#define JANIS_CASE(TI, TO) \
    return launch_kernel("rmsnorm", rmsnorm_kernel<TI, TO>, grid, block, 0, stream, 1, (const TI*)x, w, rows, (TO*)y, H, eps)
    if (x_dtype == JANIS_F32 && y_dtype == JANIS_F32) JANIS_CASE(float, float);
    if (x_dtype == JANIS_F32 && y_dtype == JANIS_BF16) JANIS_CASE(float, bf16);
    if (x_dtype == JANIS_BF16 && y_dtype == JANIS_F32) JANIS_CASE(bf16, float);
    if (x_dtype == JANIS_BF16 && y_dtype == JANIS_BF16) JANIS_CASE(bf16, bf16);
#undef JANIS_CASE
    return fail("rmsnorm: unknown dtypes %d -> %d", x_dtype, y_dtype);
}

template <typename TR, typename TO>
static int launch_add_rmsnorm(float* h, const TR* res, int n_part, size_t part_stride, const float* w_post, float eps_post,
                              const float* w_next, float eps_next, TO* y, int R, int H, cudaStream_t stream) {
    // rows of up to 8192 elements, a multiple of 8, stay in registers (each input read once, 16-byte
    // accesses); other rows take three passes
    const uintptr_t all = (uintptr_t)h | (uintptr_t)res | (uintptr_t)w_post | (uintptr_t)w_next | (uintptr_t)y |
                          (uintptr_t)(part_stride * sizeof(TR));
    if (H % 8 == 0 && H <= 8192 && (all & 15) == 0) {
        // few rows (decoding): the weights are asked for with the row, the least latency; many: fewer registers,
        // more rows an SM (measured at 2048 x 2304 in a replayed graph: 14.0 us against 16.2 with 256 threads a row)
        const bool many = R >= 256;
        const int nt = 128;
        const int need = (H / 8 + nt - 1) / nt;
#define JANIS_VEC(VPT, NT, HOIST)                                                                                       \
    return launch_kernel("add_rmsnorm", add_rmsnorm_vec_kernel<TR, TO, VPT, NT, HOIST>, dim3(R), dim3(NT), 0, stream, 1, h, \
                         res, n_part, part_stride, w_post, eps_post, w_next, eps_next, y, H)
        if (many) {
            if (need <= 1) JANIS_VEC(1, 128, false);
            if (need <= 2) JANIS_VEC(2, 128, false);
            if (need <= 3) JANIS_VEC(3, 128, false);
            if (need <= 4) JANIS_VEC(4, 128, false);
            if (need <= 6) JANIS_VEC(6, 128, false);
            JANIS_VEC(8, 128, false);
        }
        if (need <= 1) JANIS_VEC(1, 128, true);
        if (need <= 2) JANIS_VEC(2, 128, true);
        if (need <= 3) JANIS_VEC(3, 128, true);
        if (need <= 4) JANIS_VEC(4, 128, true);
        if (need <= 6) JANIS_VEC(6, 128, false);
        JANIS_VEC(8, 128, false);
#undef JANIS_VEC
    }
    return launch_kernel("add_rmsnorm", add_rmsnorm_kernel<TR, TO>, dim3(R), dim3(row_threads(H)), 0, stream, 1, h, res,
                         n_part, part_stride, w_post, eps_post, w_next, eps_next, y, H);
}

JANIS_EXPORT int janis_add_rmsnorm(float* h, const void* res, int res_dtype, int n_part, long long part_stride,
                                   const float* w_post, float eps_post, const float* w_next, float eps_next,
                                   void* y, int y_dtype, int R, int H, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (n_part < 1) return fail("add_rmsnorm: n_part must be >= 1");
    if (w_next != nullptr && y == nullptr) return fail("add_rmsnorm: a next norm needs an output");
#define JANIS_CASE(TR, TO)                                                                                        \
    return launch_add_rmsnorm<TR, TO>(h, (const TR*)res, n_part, (size_t)part_stride, w_post, eps_post, w_next,    \
                                      eps_next, (TO*)y, R, H, stream)
    if (res_dtype == JANIS_F32 && y_dtype == JANIS_F32) JANIS_CASE(float, float);
    if (res_dtype == JANIS_F32 && y_dtype == JANIS_BF16) JANIS_CASE(float, bf16);
    if (res_dtype == JANIS_BF16 && y_dtype == JANIS_F32) JANIS_CASE(bf16, float);
    if (res_dtype == JANIS_BF16 && y_dtype == JANIS_BF16) JANIS_CASE(bf16, bf16);
#undef JANIS_CASE
    return fail("add_rmsnorm: unknown dtypes %d -> %d", res_dtype, y_dtype);
}

JANIS_EXPORT int janis_gated_act(const void* gu, void* out, int dtype, int rows, int I, int group, int act,
                                 cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (group <= 0 || I % group) return fail("gated_act: width %d is not a multiple of the group %d", I, group);
    const size_t n = (size_t)rows * I;
    const int nt = 256;
    const int nb = (int)((n + nt - 1) / nt < 148 * 16 ? (n + nt - 1) / nt : 148 * 16);
    if (dtype == JANIS_F32)
        return launch_kernel("gated_act", gated_act_kernel<float>, dim3(nb), dim3(nt), 0, stream, 1, (const float*)gu,
                             (float*)out, rows, I, group, act);
    if (dtype == JANIS_BF16 && group == 8 && (((uintptr_t)gu | (uintptr_t)out) & 15) == 0) {
        const size_t n_groups = n / 8;        // rows * I / 8: group q of a row-major [rows, 2I] starts at 16 q
        const size_t want = (n_groups + nt - 1) / nt;
        const dim3 grid((int)(want < 148 * 32 ? want : 148 * 32));
        if (act == 0)
            return launch_kernel("gated_act", gated_act8_bf16_kernel<0>, grid, dim3(nt), 0, stream, 1, (const bf16*)gu,
                                 (bf16*)out, n_groups);
        return launch_kernel("gated_act", gated_act8_bf16_kernel<1>, grid, dim3(nt), 0, stream, 1, (const bf16*)gu,
                             (bf16*)out, n_groups);
    }
    if (dtype == JANIS_BF16)
        return launch_kernel("gated_act", gated_act_kernel<bf16>, dim3(nb), dim3(nt), 0, stream, 1, (const bf16*)gu,
                             (bf16*)out, rows, I, group, act);
    return fail("gated_act: unknown dtype %d", dtype);
}

JANIS_EXPORT int janis_softcap(float* x, long long n, float cap, cudaStream_t stream) {
    if (n <= 0 || !(cap > 0.f)) return 0;
    const int nt = 256;
    const long long want = (n + nt - 1) / nt;
    return launch_kernel("softcap", softcap_kernel, dim3((int)(want < 148 * 32 ? want : 148 * 32)), dim3(nt), 0, stream, 1,
                         x, (size_t)n, cap);
}

JANIS_EXPORT int janis_rope_store(void* qkv, int dtype, const int* tok_pos, const int* tok_seq,
                                  const int* seq_slot, const int* seq_end, const float* inv_freq, int rot,
                                  int T, int nq, int nkv, int hd, int row_heads, void* kpool, void* vpool,
                                  const int* page_table, int table_stride, int ring_len, int store_q_only,
                                  cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rot < 0 || rot > hd || (rot & 1)) return fail("rope_store: rotary width %d does not fit head size %d", rot, hd);
    if (row_heads < (store_q_only ? nq : nq + 2 * nkv)) return fail("rope_store: rows of %d heads are too short", row_heads);
    if (ring_len % JANIS_PAGE) return fail("rope_store: ring length %d is not a multiple of the page", ring_len);
    const int heads = store_q_only ? nq : nq + 2 * nkv;
    const uintptr_t all = (uintptr_t)qkv | (uintptr_t)kpool | (uintptr_t)vpool;
    if (rot == hd && hd % 16 == 0 && (all & 15) == 0) {
        // 16-byte accesses; few tokens: a thread per head, many: 4 heads per thread, which share the angles
        const int per = (long long)T * heads >= 4096 ? 4 : 1;
        const long long units = (long long)T * ((heads + per - 1) / per) * (hd / 16);
        const dim3 grid((unsigned)((units + 127) / 128)), block(128);
        if (dtype == JANIS_F32)
            return launch_kernel("rope_store", rope_store_vec_kernel<float>, grid, block, 0, stream, 1, (float*)qkv, tok_pos,
                                 tok_seq, seq_slot, seq_end, inv_freq, T, nq, nkv, hd, row_heads, (float*)kpool,
                                 (float*)vpool, page_table, table_stride, ring_len, heads, per);
        if (dtype == JANIS_BF16)
            return launch_kernel("rope_store", rope_store_vec_kernel<bf16>, grid, block, 0, stream, 1, (bf16*)qkv, tok_pos,
                                 tok_seq, seq_slot, seq_end, inv_freq, T, nq, nkv, hd, row_heads, (bf16*)kpool, (bf16*)vpool,
                                 page_table, table_stride, ring_len, heads, per);
        return fail("rope_store: unknown dtype %d", dtype);
    }
    // partial rotary widths and odd sizes: element by element; few tokens: a CTA per head, many: up to 4 heads per CTA
    int per = (int)(((long long)T * heads) / 2048);
    per = per < 1 ? 1 : (per > 4 ? 4 : per);
    const int want = rot < hd ? hd : hd / 2;                 // threads that have an element of their own
    const int nt = want >= 256 ? 256 : ((want + 31) / 32) * 32;
    const dim3 grid(T, (heads + per - 1) / per), block(nt < 32 ? 32 : nt);
    if (dtype == JANIS_F32)
        return launch_kernel("rope_store", rope_store_kernel<float>, grid, block, 0, stream, 1, (float*)qkv, tok_pos, tok_seq,
                             seq_slot, seq_end, inv_freq, rot, nq, nkv, hd, row_heads, (float*)kpool, (float*)vpool,
                             page_table, table_stride, ring_len, heads, per);
    if (dtype == JANIS_BF16)
        return launch_kernel("rope_store", rope_store_kernel<bf16>, grid, block, 0, stream, 1, (bf16*)qkv, tok_pos, tok_seq,
                             seq_slot, seq_end, inv_freq, rot, nq, nkv, hd, row_heads, (bf16*)kpool, (bf16*)vpool,
                             page_table, table_stride, ring_len, heads, per);
    return fail("rope_store: unknown dtype %d", dtype);
}

JANIS_EXPORT int janis_kv_store(const void* qkv, int dtype, const int* tok_pos, const int* tok_seq, const int* seq_slot,
                                const int* seq_end, int T, int nq, int nkv, int hd, int row_heads, void* kpool,
                                void* vpool, const int* page_table, int table_stride, int ring_len, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (row_heads < nq + 2 * nkv) return fail("kv_store: rows of %d heads are too short", row_heads);
    if (ring_len % JANIS_PAGE) return fail("kv_store: ring length %d is not a multiple of the page", ring_len);
    if (((uintptr_t)qkv | (uintptr_t)kpool | (uintptr_t)vpool) & 15) return fail("kv_store: operands must be 16-byte aligned");
    const int vec = dtype == JANIS_F32 ? 4 : 8;
    if (hd % vec) return fail("kv_store: head size %d is not a multiple of %d", hd, vec);
    const long long units = (long long)T * 2 * nkv * (hd / vec);
    const dim3 grid((unsigned)((units + 255) / 256)), block(256);
    if (dtype == JANIS_F32)
        return launch_kernel("kv_store", kv_store_kernel<float>, grid, block, 0, stream, 1, (const float*)qkv, tok_pos, tok_seq,
                             seq_slot, seq_end, T, nq, nkv, hd, row_heads, (float*)kpool, (float*)vpool, page_table,
                             table_stride, ring_len);
    if (dtype == JANIS_BF16)
        return launch_kernel("kv_store", kv_store_kernel<bf16>, grid, block, 0, stream, 1, (const bf16*)qkv, tok_pos, tok_seq,
                             seq_slot, seq_end, T, nq, nkv, hd, row_heads, (bf16*)kpool, (bf16*)vpool, page_table,
                             table_stride, ring_len);
    return fail("kv_store: unknown dtype %d", dtype);
}

JANIS_EXPORT const char* janis_last_error() { return error_buffer(); }
