// Softmax attention for one head size (JANIS_HEAD_DIM, fixed when this file is
// compiled; the library is built once per head size a model needs).
//
//   prefill: packed sequences of unequal lengths that start at position 0; a
//            query sees the keys of its own sequence up to itself and, with a
//            window, only the last `window` of them.  Keys and values are read
//            from the step's own [T, nq + 2 nkv, hd] buffer.
//   decode : one query per sequence over the paged cache (a ring for windowed
//            layers), the key range cut into chunks that separate CTAs reduce;
//            a second kernel merges the chunks in ascending order.
//
// Scores are q.k * scale, then cap * tanh(s / cap) when a cap is given, then the
// mask, then softmax; all of it and the weighted sum of values in float.  Query
// heads that share a key/value head are handled together so that keys and values
// are read once.  A group of LPK lanes owns one key at a time (16-byte loads);
// the lane groups of a warp, and the warps of a CTA, keep running maxima and sums
// of their own and are merged in a fixed order at the end.
#include "common.cuh"

#ifndef JANIS_HEAD_DIM
#error "compile with -DJANIS_HEAD_DIM=<head size, a multiple of 16>"
#endif
#if (JANIS_HEAD_DIM % 16) != 0 || JANIS_HEAD_DIM < 16 || JANIS_HEAD_DIM > 512
#error "head size must be a multiple of 16 between 16 and 512"
#endif

namespace janis {

constexpr int HD = JANIS_HEAD_DIM;
constexpr int ATTN_WARPS = 4;

constexpr int pow2_divisor_up_to_8(int n) { return n % 8 == 0 ? 8 : (n % 4 == 0 ? 4 : (n % 2 == 0 ? 2 : 1)); }
constexpr int clamp_int(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

template <typename T> struct Geo {
    static constexpr int VEC = Vec16<T>::N;                 // elements in 16 bytes
    static constexpr int NCHUNK = HD / VEC;                 // 16-byte pieces of a key
    static constexpr int LPK = pow2_divisor_up_to_8(NCHUNK);  // lanes that share a key
    static constexpr int CPL = NCHUNK / LPK;                // pieces per lane
    static constexpr int EPL = CPL * VEC;                   // elements per lane
    static constexpr int KPW = 32 / LPK;                    // keys a warp handles at a time
    static constexpr int RG = clamp_int(64 / EPL, 1, 8);    // query heads handled together
};

template <typename T> struct Lane {
    typedef Geo<T> G;
    float q[G::RG][G::EPL];
    float acc[G::RG][G::EPL];
    float m[G::RG], l[G::RG];

    __device__ __forceinline__ void init() {
#pragma unroll
        for (int r = 0; r < G::RG; ++r) {
            m[r] = -INFINITY;
            l[r] = 0.f;
#pragma unroll
            for (int e = 0; e < G::EPL; ++e) acc[r][e] = 0.f;
        }
    }

    // q of head `head` (or zeros), times `scale`
    __device__ __forceinline__ void load_q(const T* qrow, int r, bool valid, float scale, int lig) {
#pragma unroll
        for (int c = 0; c < G::CPL; ++c) {
            float f[G::VEC];
            if (valid) Vec16<T>::load(qrow + (c * G::LPK + lig) * G::VEC, f);
#pragma unroll
            for (int e = 0; e < G::VEC; ++e) q[r][c * G::VEC + e] = valid ? f[e] * scale : 0.f;
        }
    }

    // One key for this lane group.  Every lane of the warp must call this together
    // (the reduction uses full-warp shuffles); `valid` says whether the key counts.
    __device__ __forceinline__ void key(const T* kp, const T* vp, bool valid, float cap, int lig) {
        float kf[G::EPL];
#pragma unroll
        for (int c = 0; c < G::CPL; ++c) {
            if (valid) Vec16<T>::load(kp + (c * G::LPK + lig) * G::VEC, kf + c * G::VEC);
            else {
#pragma unroll
                for (int e = 0; e < G::VEC; ++e) kf[c * G::VEC + e] = 0.f;
            }
        }
        float s[G::RG];
#pragma unroll
        for (int r = 0; r < G::RG; ++r) {
            float d = 0.f;
#pragma unroll
            for (int e = 0; e < G::EPL; ++e) d = fmaf(q[r][e], kf[e], d);
#pragma unroll
            for (int o = G::LPK / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
            s[r] = d;
        }
        if (!valid) return;
        float vf[G::EPL];
#pragma unroll
        for (int c = 0; c < G::CPL; ++c) Vec16<T>::load(vp + (c * G::LPK + lig) * G::VEC, vf + c * G::VEC);
#pragma unroll
        for (int r = 0; r < G::RG; ++r) {
            float sc = s[r];
            if (cap > 0.f) sc = cap * tanhf(sc / cap);
            const float mn = fmaxf(m[r], sc);
            const float corr = expf(m[r] - mn);     // m = -inf at first: exp(-inf) = 0
            const float p = expf(sc - mn);
            l[r] = l[r] * corr + p;
#pragma unroll
            for (int e = 0; e < G::EPL; ++e) acc[r][e] = fmaf(p, vf[e], acc[r][e] * corr);
            m[r] = mn;
        }
    }

    // Fold the lane groups of the warp into every group (butterfly over groups).
    __device__ __forceinline__ void merge_groups() {
#pragma unroll
        for (int o = G::LPK; o < 32; o <<= 1) {
#pragma unroll
            for (int r = 0; r < G::RG; ++r) {
                const float mo = __shfl_xor_sync(0xffffffffu, m[r], o);
                const float lo = __shfl_xor_sync(0xffffffffu, l[r], o);
                const float mn = fmaxf(m[r], mo);
                const float a = m[r] == -INFINITY ? 0.f : expf(m[r] - mn);
                const float b = mo == -INFINITY ? 0.f : expf(mo - mn);
                l[r] = l[r] * a + lo * b;
#pragma unroll
                for (int e = 0; e < G::EPL; ++e) {
                    const float ao = __shfl_xor_sync(0xffffffffu, acc[r][e], o);
                    acc[r][e] = acc[r][e] * a + ao * b;
                }
                m[r] = mn;
            }
        }
    }
};

// ---------------------------------------------------------------------------
// prefill: one warp per (token, key/value head, group of query heads)
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(ATTN_WARPS * 32)
attn_prefill_kernel(const T* __restrict__ qkv, const T* __restrict__ kv_src, const int* __restrict__ tok_pos,
                    const int* __restrict__ tok_seq, const int* __restrict__ seq_first_row,
                    T* __restrict__ out, int n_tok, int nq, int nkv, int q_row_heads, int kv_row_heads,
                    int kv_k_head0, float scale, float cap, int window) {
    typedef Geo<T> G;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * ATTN_WARPS + warp;
    if (t >= n_tok) return;
    const int rep = nq / nkv;
    const int groups = (rep + G::RG - 1) / G::RG;
    const int kvh = blockIdx.y / groups, hg = blockIdx.y % groups;
    const int h0 = kvh * rep + hg * G::RG;
    const int nh_here = min(G::RG, rep - hg * G::RG);
    const int lig = lane % G::LPK, grp = lane / G::LPK;
    const int pos = tok_pos[t];
    const int first = seq_first_row[tok_seq[t]];         // row of this sequence's position 0
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;

    Lane<T> st;
    st.init();
    const T* qrow = qkv + (size_t)t * q_row_heads * HD;
#pragma unroll
    for (int r = 0; r < G::RG; ++r) st.load_q(qrow + (size_t)(h0 + r) * HD, r, r < nh_here, scale, lig);

    // keys and values of position j: row first + j of kv_src, heads k0 + kvh and k0 + nkv + kvh
    const size_t row_elems = (size_t)kv_row_heads * HD;
    for (int j0 = lo; j0 <= pos; j0 += G::KPW) {
        const int j = j0 + grp;
        const bool valid = j <= pos;
        const T* base = kv_src + (size_t)(first + (valid ? j : pos)) * row_elems;
        st.key(base + (size_t)(kv_k_head0 + kvh) * HD, base + (size_t)(kv_k_head0 + nkv + kvh) * HD, valid, cap,
               lig);
    }
    st.merge_groups();
    if (grp != 0) return;
#pragma unroll
    for (int r = 0; r < G::RG; ++r) {
        if (r >= nh_here) continue;
        const float inv = 1.0f / st.l[r];
        T* o = out + (size_t)t * nq * HD + (size_t)(h0 + r) * HD;
#pragma unroll
        for (int c = 0; c < G::CPL; ++c) {
            float f[G::VEC];
#pragma unroll
            for (int e = 0; e < G::VEC; ++e) f[e] = st.acc[r][c * G::VEC + e] * inv;
            Vec16<T>::store(o + (c * G::LPK + lig) * G::VEC, f);
        }
    }
}

// ---------------------------------------------------------------------------
// decode: grid (chunk, key/value head x head group, sequence)
// partial layout: [seq, head, chunk slot, 2 + HD] = (max, sum, unnormalised values)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void chunk_range(int len, int window, int chunk, int& lo, int& first_chunk,
                                            int& n_chunks) {
    lo = window > 0 ? max(0, len - window) : 0;
    first_chunk = lo / chunk;
    n_chunks = (len + chunk - 1) / chunk - first_chunk;
}

template <typename T>
__global__ void __launch_bounds__(ATTN_WARPS * 32)
attn_decode_kernel(const T* __restrict__ qkv, const T* __restrict__ kpool, const T* __restrict__ vpool,
                   const int* __restrict__ page_table, int table_stride, const int* __restrict__ seq_slot,
                   const int* __restrict__ seq_len, float* __restrict__ partial, int nq, int nkv,
                   int q_row_heads, float scale, float cap, int window, int ring_len, int chunk) {
    typedef Geo<T> G;
    __shared__ float sm[ATTN_WARPS][G::RG][HD + 2];
    const int s = blockIdx.z;
    const int slot = seq_slot[s];
    if (slot < 0) return;
    const int len = seq_len[s];
    int lo, first_chunk, n_chunks;
    chunk_range(len, window, chunk, lo, first_chunk, n_chunks);
    if ((int)blockIdx.x >= n_chunks) return;
    const int c = first_chunk + blockIdx.x;
    const int k_begin = max(lo, c * chunk), k_end = min(len, (c + 1) * chunk);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rep = nq / nkv;
    const int groups = (rep + G::RG - 1) / G::RG;
    const int kvh = blockIdx.y / groups, hg = blockIdx.y % groups;
    const int h0 = kvh * rep + hg * G::RG;
    const int nh_here = min(G::RG, rep - hg * G::RG);
    const int lig = lane % G::LPK, grp = lane / G::LPK;

    Lane<T> st;
    st.init();
    const T* qrow = qkv + (size_t)s * q_row_heads * HD;
#pragma unroll
    for (int r = 0; r < G::RG; ++r) st.load_q(qrow + (size_t)(h0 + r) * HD, r, r < nh_here, scale, lig);

    const int* table = page_table + (size_t)slot * table_stride;
    for (int j0 = k_begin + warp * G::KPW; j0 < k_end; j0 += ATTN_WARPS * G::KPW) {
        const int j = j0 + grp;
        const bool valid = j < k_end;
        const int idx = ring_len > 0 ? (valid ? j : k_begin) % ring_len : (valid ? j : k_begin);
        const int page = table[idx / JANIS_PAGE];
        const size_t off = (((size_t)page * nkv + kvh) * JANIS_PAGE + idx % JANIS_PAGE) * HD;
        st.key(kpool + off, vpool + off, valid, cap, lig);
    }
    st.merge_groups();
    if (grp == 0) {
#pragma unroll
        for (int r = 0; r < G::RG; ++r) {
            if (lig == 0) { sm[warp][r][0] = st.m[r]; sm[warp][r][1] = st.l[r]; }
#pragma unroll
            for (int cc = 0; cc < G::CPL; ++cc)
#pragma unroll
                for (int e = 0; e < G::VEC; ++e)
                    sm[warp][r][2 + (cc * G::LPK + lig) * G::VEC + e] = st.acc[r][cc * G::VEC + e];
        }
    }
    __syncthreads();
    const int max_chunks = gridDim.x;
    for (int idx = threadIdx.x; idx < nh_here * (HD + 2); idx += blockDim.x) {
        const int r = idx / (HD + 2), d = idx % (HD + 2);
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < ATTN_WARPS; ++w) mx = fmaxf(mx, sm[w][r][0]);
        float v;
        if (d == 0) v = mx;
        else {
            v = 0.f;
#pragma unroll
            for (int w = 0; w < ATTN_WARPS; ++w) {
                const float mw = sm[w][r][0];
                if (mw != -INFINITY) v += sm[w][r][d] * expf(mw - mx);
            }
        }
        partial[(((size_t)s * nq + h0 + r) * max_chunks + blockIdx.x) * (HD + 2) + d] = v;
    }
}

template <typename T>
__global__ void attn_merge_kernel(const float* __restrict__ partial, const int* __restrict__ seq_slot,
                                  const int* __restrict__ seq_len, T* __restrict__ out, int nq, int max_chunks,
                                  int window, int chunk) {
    const int s = blockIdx.x, h = blockIdx.y;
    T* o = out + ((size_t)s * nq + h) * HD;
    if (seq_slot[s] < 0) {
        for (int d = threadIdx.x; d < HD; d += blockDim.x) o[d] = from_float<T>(0.f);
        return;
    }
    int lo, first_chunk, n_chunks;
    chunk_range(seq_len[s], window, chunk, lo, first_chunk, n_chunks);
    if (n_chunks > max_chunks) {   // the launch was sized for shorter sequences: make it visible
        for (int d = threadIdx.x; d < HD; d += blockDim.x) o[d] = from_float<T>(__int_as_float(0x7fc00000));
        return;
    }
    const float* p = partial + ((size_t)s * nq + h) * max_chunks * (HD + 2);
    float mx = -INFINITY;
    for (int c = 0; c < n_chunks; ++c) mx = fmaxf(mx, p[(size_t)c * (HD + 2)]);
    float l = 0.f;
    for (int c = 0; c < n_chunks; ++c) {
        const float mc = p[(size_t)c * (HD + 2)];
        if (mc != -INFINITY) l += p[(size_t)c * (HD + 2) + 1] * expf(mc - mx);
    }
    const float inv = 1.0f / l;
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float a = 0.f;
        for (int c = 0; c < n_chunks; ++c) {
            const float mc = p[(size_t)c * (HD + 2)];
            if (mc != -INFINITY) a += p[(size_t)c * (HD + 2) + 2 + d] * expf(mc - mx);
        }
        o[d] = from_float<T>(a * inv);
    }
}

}  // namespace janis

using namespace janis;

JANIS_EXPORT int janis_attn_head_dim() { return HD; }

// floats of scratch that a decode call with these sizes needs
JANIS_EXPORT long long janis_attn_decode_scratch(int n_seq, int nq, int max_chunks) {
    return (long long)n_seq * nq * max_chunks * (HD + 2);
}

// qkv: [T, q_row_heads, hd] holds the queries in its first nq heads; keys and values of position j of a
// sequence are read from row (seq_first_row + j) of kv_src, a [rows, kv_row_heads, hd]
// buffer whose key heads start at head kv_k_head0 and value heads nkv later
// (kv_src = qkv, kv_row_heads = nq + 2 nkv, kv_k_head0 = nq for a layer's own keys).
JANIS_EXPORT int janis_attn_prefill(const void* qkv, const void* kv_src, int dtype, const int* tok_pos,
                                    const int* tok_seq, const int* seq_first_row, void* out, int n_tok, int nq,
                                    int nkv, int q_row_heads, int kv_row_heads, int kv_k_head0, float scale,
                                    float cap, int window, cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    if (nkv <= 0 || nq % nkv) return fail("attn_prefill: %d query heads do not divide over %d key heads", nq, nkv);
    const int rep = nq / nkv;
    dim3 grid((n_tok + ATTN_WARPS - 1) / ATTN_WARPS, 1, 1);
    if (dtype == JANIS_F32) {
        grid.y = nkv * ((rep + Geo<float>::RG - 1) / Geo<float>::RG);
        attn_prefill_kernel<float><<<grid, ATTN_WARPS * 32, 0, stream>>>(
            (const float*)qkv, (const float*)kv_src, tok_pos, tok_seq, seq_first_row, (float*)out, n_tok, nq, nkv,
            q_row_heads, kv_row_heads, kv_k_head0, scale, cap, window);
    } else if (dtype == JANIS_BF16) {
        grid.y = nkv * ((rep + Geo<bf16>::RG - 1) / Geo<bf16>::RG);
        attn_prefill_kernel<bf16><<<grid, ATTN_WARPS * 32, 0, stream>>>(
            (const bf16*)qkv, (const bf16*)kv_src, tok_pos, tok_seq, seq_first_row, (bf16*)out, n_tok, nq, nkv,
            q_row_heads, kv_row_heads, kv_k_head0, scale, cap, window);
    } else {
        return fail("attn_prefill: unknown dtype %d", dtype);
    }
    return launched("attn_prefill");
}

JANIS_EXPORT int janis_attn_decode(const void* qkv, const void* kpool, const void* vpool, int dtype,
                                   const int* page_table, int table_stride, const int* seq_slot,
                                   const int* seq_len, float* partial, long long partial_floats, void* out,
                                   int n_seq, int nq, int nkv, int q_row_heads, float scale, float cap, int window,
                                   int ring_len, int chunk, int max_chunks, cudaStream_t stream) {
    if (n_seq <= 0) return 0;
    if (nkv <= 0 || nq % nkv) return fail("attn_decode: %d query heads do not divide over %d key heads", nq, nkv);
    if (chunk <= 0 || chunk % JANIS_PAGE) return fail("attn_decode: chunk %d is not a multiple of the page", chunk);
    if (ring_len % JANIS_PAGE) return fail("attn_decode: ring length %d is not a multiple of the page", ring_len);
    if (ring_len > 0 && (window <= 0 || window > ring_len))
        return fail("attn_decode: window %d does not fit its ring of %d", window, ring_len);
    if (max_chunks <= 0) return fail("attn_decode: max_chunks must be positive");
    if (partial_floats < janis_attn_decode_scratch(n_seq, nq, max_chunks))
        return fail("attn_decode: scratch of %lld floats is too small, %lld needed", partial_floats,
                    janis_attn_decode_scratch(n_seq, nq, max_chunks));
    if (n_seq > 65535) return fail("attn_decode: too many sequences (%d)", n_seq);
    const int rep = nq / nkv;
    dim3 mgrid(n_seq, nq);
    const int mthreads = HD < 256 ? (HD < 32 ? 32 : HD) : 256;
    if (dtype == JANIS_F32) {
        dim3 grid(max_chunks, nkv * ((rep + Geo<float>::RG - 1) / Geo<float>::RG), n_seq);
        attn_decode_kernel<float><<<grid, ATTN_WARPS * 32, 0, stream>>>(
            (const float*)qkv, (const float*)kpool, (const float*)vpool, page_table, table_stride, seq_slot, seq_len,
            partial, nq, nkv, q_row_heads, scale, cap, window, ring_len, chunk);
        if (launched("attn_decode")) return 1;
        attn_merge_kernel<float><<<mgrid, mthreads, 0, stream>>>(partial, seq_slot, seq_len, (float*)out, nq,
                                                                  max_chunks, window, chunk);
    } else if (dtype == JANIS_BF16) {
        dim3 grid(max_chunks, nkv * ((rep + Geo<bf16>::RG - 1) / Geo<bf16>::RG), n_seq);
        attn_decode_kernel<bf16><<<grid, ATTN_WARPS * 32, 0, stream>>>(
            (const bf16*)qkv, (const bf16*)kpool, (const bf16*)vpool, page_table, table_stride, seq_slot, seq_len,
            partial, nq, nkv, q_row_heads, scale, cap, window, ring_len, chunk);
        if (launched("attn_decode")) return 1;
        attn_merge_kernel<bf16><<<mgrid, mthreads, 0, stream>>>(partial, seq_slot, seq_len, (bf16*)out, nq,
                                                                 max_chunks, window, chunk);
    } else {
        return fail("attn_decode: unknown dtype %d", dtype);
    }
    return launched("attn_merge");
}

JANIS_EXPORT const char* janis_last_error() { return error_buffer(); }
