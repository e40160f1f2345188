// Softmax attention for one head size (JANIS_HEAD_DIM, fixed when this file is
// compiled; the library is built once per head size a model needs).
//
//   prefill: packed sequences of unequal lengths; a query sees the keys of its
//            own sequence up to itself and, with a window, only the last `window`
//            of them.  Keys and values of the step's own positions are read from
//            the step's [T, nq + 2 nkv, hd] buffer, those of positions that earlier
//            steps stored (a prompt that comes in several steps) from the cache.
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

constexpr int pow2_divisor_up_to(int n, int cap) {
    return (cap >= 16 && n % 16 == 0) ? 16 : (n % 8 == 0 ? 8 : (n % 4 == 0 ? 4 : (n % 2 == 0 ? 2 : 1)));
}
constexpr int clamp_int(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

template <typename T, int LMAX = 8, int BUDGET = 64> struct Geo {
    static constexpr int VEC = Vec16<T>::N;                 // elements in 16 bytes
    static constexpr int NCHUNK = HD / VEC;                 // 16-byte pieces of a key
    static constexpr int LPK = pow2_divisor_up_to(NCHUNK, LMAX);  // lanes that share a key (at most LMAX)
    static constexpr int CPL = NCHUNK / LPK;                // pieces per lane
    static constexpr int EPL = CPL * VEC;                   // elements per lane
    static constexpr int KPW = 32 / LPK;                    // keys a warp handles at a time
    static constexpr int RG = clamp_int(BUDGET / EPL, 1, 8);  // query heads handled together (register budget)
};

template <typename T, int LMAX = 8, int BUDGET = 64> struct Lane {
    typedef Geo<T, LMAX, BUDGET> G;
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
                    int kv_k_head0, float scale, float cap, int window, CachedPrefix cached) {
    typedef Geo<T> G;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * ATTN_WARPS + warp;
    grid_dependents_launch();
    grid_dependency_wait();
    if (t >= n_tok) return;
    const int rep = nq / nkv;
    const int groups = (rep + G::RG - 1) / G::RG;
    const int kvh = blockIdx.y / groups, hg = blockIdx.y % groups;
    const int h0 = kvh * rep + hg * G::RG;
    const int nh_here = min(G::RG, rep - hg * G::RG);
    const int lig = lane % G::LPK, grp = lane / G::LPK;
    const int pos = tok_pos[t];
    const int seq = tok_seq[t];
    const int start = cached.seq_start ? cached.seq_start[seq] : 0;   // positions below it are in the cache
    const int slot = cached.seq_start ? cached.seq_slot[seq] : -1;
    const int first = seq_first_row[seq] - start;        // row that position 0 would have in the step's buffer
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
        const T* base = kv_src + (size_t)(first + (valid && j >= start ? j : pos)) * row_elems;
        const T* kp = base + (size_t)(kv_k_head0 + kvh) * HD;
        const T* vp = base + (size_t)(kv_k_head0 + nkv + kvh) * HD;
        if (valid && j < start && slot >= 0) {            // stored by an earlier step
            const size_t off = cached_row(cached, slot, j, nkv, kvh, HD);
            kp = (const T*)cached.kpool + off;
            vp = (const T*)cached.vpool + off;
        }
        st.key(kp, vp, valid, cap, lig);                  // (one call for the whole warp: it shuffles)
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

// What a decode CTA leaves for the merge: the warps' states folded in warp order.
template <typename T, int LMAX, int BUDGET, int WARPS>
__device__ __forceinline__ void write_partial(Lane<T, LMAX, BUDGET>& st, float (*sm)[Geo<T, LMAX, BUDGET>::RG][HD + 2],
                                              float* __restrict__ partial, int s, int nq, int h0, int nh_here, int warp,
                                              int lig, int grp) {
    typedef Geo<T, LMAX, BUDGET> G;
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
        for (int w = 0; w < WARPS; ++w) mx = fmaxf(mx, sm[w][r][0]);
        float v;
        if (d == 0) v = mx;
        else {
            v = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const float mw = sm[w][r][0];
                if (mw != -INFINITY) v += sm[w][r][d] * expf(mw - mx);
            }
        }
        partial[(((size_t)s * nq + h0 + r) * max_chunks + blockIdx.x) * (HD + 2) + d] = v;
    }
}

// Decode attention, keys and values read straight from global memory into registers.
template <typename T>
__global__ void __launch_bounds__(ATTN_WARPS * 32)
attn_decode_kernel(const T* __restrict__ qkv, const T* __restrict__ kpool, const T* __restrict__ vpool,
                   const int* __restrict__ page_table, int table_stride, const int* __restrict__ seq_slot,
                   const int* __restrict__ seq_len, float* __restrict__ partial, int nq, int nkv,
                   int q_row_heads, float scale, float cap, int window, int ring_len, int chunk) {
    typedef Geo<T> G;
    __shared__ float sm[ATTN_WARPS][G::RG][HD + 2];
    const int s = blockIdx.z;
    grid_dependents_launch();
    grid_dependency_wait();
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
    write_partial<T, 8, 64, ATTN_WARPS>(st, sm, partial, s, nq, h0, nh_here, warp, lig, grp);
}

// ---------------------------------------------------------------------------
// The same step with keys and values staged through shared memory by the TMA
// engine: one thread issues bulk copies (cp.async.bulk) of whole tiles of a
// cache page, three stages deep, and an mbarrier per stage tells the warps when
// the bytes have landed.  A (page, head) of the cache is contiguous, so a tile of
// TILE keys is one copy of TILE * hd elements for keys and one for values.  The
// register kernel above keeps ~16 KB in flight per SM and is bound by latency;
// this one keeps up to 3 stages per CTA in flight.
// Every wait is bounded: a barrier that does not complete makes the CTA give up,
// count the event in g_wait_timeouts and return (its output is then garbage and the
// host finds the count in janis_attn_wait_timeouts()).
// ---------------------------------------------------------------------------
__device__ int g_wait_timeouts = 0;

constexpr int pow2_floor(int n) { return n >= 64 ? 64 : (n >= 32 ? 32 : (n >= 16 ? 16 : (n >= 8 ? 8 : (n >= 4 ? 4 : (n >= 2 ? 2 : 1))))); }
constexpr int max_int(int a, int b) { return a > b ? a : b; }
constexpr int pow2_ceil(int n) { return n <= 1 ? 1 : (n <= 2 ? 2 : (n <= 4 ? 4 : (n <= 8 ? 8 : (n <= 16 ? 16 : 32)))); }

#ifndef JANIS_STAGES
#define JANIS_STAGES 3            // stages of the bulk-copy pipeline
#endif
#ifndef JANIS_STAGE_BUDGET
#define JANIS_STAGE_BUDGET 32768  // bytes of keys and values a stage aims at
#endif

template <typename T> struct Staged {
    static constexpr int STAGES = JANIS_STAGES;
    static constexpr int LMAX = 16, BUDGET = 32;
    static constexpr int SMEM_LIMIT = 200 * 1024;
    // a pass never exceeds a page; head sizes whose keys split over few lanes (many keys a warp) take fewer warps,
    // so that the stages still fit shared memory
    static constexpr int fit_warps() {
        int w = clamp_int(JANIS_PAGE / Geo<T, LMAX>::KPW, 1, 8);
        while (w > 1 && STAGES * 2 * w * Geo<T, LMAX>::KPW * HD * (int)sizeof(T) > SMEM_LIMIT) w /= 2;
        return w;
    }
    static constexpr int WARPS = fit_warps();
    static constexpr int KEYS_PER_PASS = WARPS * Geo<T, LMAX>::KPW;        // keys the CTA handles at a time
    static constexpr int TILE = max_int(KEYS_PER_PASS, pow2_floor(JANIS_STAGE_BUDGET / (2 * HD * (int)sizeof(T))));
    static constexpr int TILE_BYTES = TILE * HD * (int)sizeof(T);
    static constexpr int STAGE_BYTES = 2 * TILE_BYTES;                      // keys, then values
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES;
    static_assert(TILE <= JANIS_PAGE && JANIS_PAGE % TILE == 0, "a tile must divide a page");
    static_assert(TILE % KEYS_PER_PASS == 0, "a tile must be whole passes");
    static_assert(SMEM_BYTES <= SMEM_LIMIT, "stages do not fit shared memory");
};

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, int bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, int bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
// m16n8k16 whose 16-row operand has rows 8..15 zero (a1 = a3 = 0): d += A B
__device__ __forceinline__ void mma_rows8(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    const uint32_t z = 0u;
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(z), "r"(a2), "r"(z), "r"(b0), "r"(b1));
}
// true when the phase with this parity has completed; false after a bounded number of tries
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int tries = 1 << 22) {
    for (int it = 0; it < tries; ++it) {
        uint32_t done;
        asm volatile(
            "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

// The bounded wait on its own: a barrier that nothing completes, waited for with `tries` tries.  The wait gives
// up, the kernel says so (status 1, and the counter of timeouts goes up) and returns; the context stays usable.
__global__ void wait_probe_kernel(int tries, int* __restrict__ status) {
    __shared__ __align__(8) unsigned long long never;
    const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&never);
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();
    const bool done = mbar_wait(bar, 0, tries);
    if (threadIdx.x == 0) {
        *status = done ? 0 : 1;
        if (!done) atomicAdd(&g_wait_timeouts, 1);
    }
}

template <typename T>
__global__ void __launch_bounds__(Staged<T>::WARPS * 32)
attn_decode_staged_kernel(const T* __restrict__ qkv, const T* __restrict__ kpool, const T* __restrict__ vpool,
                          const int* __restrict__ page_table, int table_stride, const int* __restrict__ seq_slot,
                          const int* __restrict__ seq_len, float* __restrict__ partial, int nq, int nkv,
                          int q_row_heads, float scale, float cap, int window, int ring_len, int chunk) {
    typedef Staged<T> S;
    typedef Geo<T, S::LMAX, S::BUDGET> G;
    extern __shared__ __align__(128) unsigned char stage_mem[];
    __shared__ __align__(8) unsigned long long full[S::STAGES];
    const int s = blockIdx.z;
    grid_dependents_launch();
    grid_dependency_wait();
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

    const uint32_t stage0 = (uint32_t)__cvta_generic_to_shared(stage_mem);
    const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(full);
    if (threadIdx.x == 0) {
        for (int i = 0; i < S::STAGES; ++i) mbar_init(bar0 + 8 * i, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    // tiles of TILE positions, aligned to TILE, that cover [k_begin, k_end)
    const int t_first = (k_begin / S::TILE) * S::TILE;
    const int n_tiles = (k_end - t_first + S::TILE - 1) / S::TILE;
    const int* table = page_table + (size_t)slot * table_stride;
    auto issue = [&](int i) {       // thread 0: bring tile i into its stage
        const int p0 = t_first + i * S::TILE;
        const int idx = ring_len > 0 ? p0 % ring_len : p0;
        const int page = table[idx / JANIS_PAGE];
        const size_t off = (((size_t)page * nkv + kvh) * JANIS_PAGE + idx % JANIS_PAGE) * HD;
        const int st_i = i % S::STAGES;
        const uint32_t dst = stage0 + st_i * S::STAGE_BYTES, bar = bar0 + 8 * st_i;
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // earlier reads of this stage are done
        mbar_expect_tx(bar, S::STAGE_BYTES);
        bulk_load(dst, kpool + off, S::TILE_BYTES, bar);
        bulk_load(dst + S::TILE_BYTES, vpool + off, S::TILE_BYTES, bar);
    };
    if (threadIdx.x == 0)
        for (int i = 0; i < S::STAGES && i < n_tiles; ++i) issue(i);

    Lane<T, S::LMAX, S::BUDGET> st;
    st.init();
    const T* qrow = qkv + (size_t)s * q_row_heads * HD;
#pragma unroll
    for (int r = 0; r < G::RG; ++r) st.load_q(qrow + (size_t)(h0 + r) * HD, r, r < nh_here, scale, lig);

    for (int i = 0; i < n_tiles; ++i) {
        const int st_i = i % S::STAGES;
        const bool landed = mbar_wait(bar0 + 8 * st_i, (i / S::STAGES) & 1);
        if (landed) {
            const T* ks = reinterpret_cast<const T*>(stage_mem + (size_t)st_i * S::STAGE_BYTES);
            const T* vs = reinterpret_cast<const T*>(stage_mem + (size_t)st_i * S::STAGE_BYTES + S::TILE_BYTES);
            const int p0 = t_first + i * S::TILE;
#pragma unroll
            for (int pass = 0; pass < S::TILE / S::KEYS_PER_PASS; ++pass) {
                const int r = pass * S::KEYS_PER_PASS + warp * G::KPW + grp;      // row of the tile
                const int j = p0 + r;
                st.key(ks + (size_t)r * HD, vs + (size_t)r * HD, j >= k_begin && j < k_end, cap, lig);
            }
        }
        // everyone has read the stage (or given up): the same barrier tells all of a timeout
        if (!__syncthreads_and(landed ? 1 : 0)) {
            if (threadIdx.x == 0) atomicAdd(&g_wait_timeouts, 1);
            return;
        }
        if (threadIdx.x == 0 && i + S::STAGES < n_tiles) issue(i + S::STAGES);
    }
    // every tile has been consumed and nothing is in flight: the stages' memory now holds the warps' states
    static_assert(sizeof(float) * S::WARPS * G::RG * (HD + 2) <= S::SMEM_BYTES, "the merge does not fit the stages");
    float (*sm)[G::RG][HD + 2] = reinterpret_cast<float (*)[G::RG][HD + 2]>(stage_mem);
    write_partial<T, S::LMAX, S::BUDGET, S::WARPS>(st, sm, partial, s, nq, h0, nh_here, warp, lig, grp);
}

// ---------------------------------------------------------------------------
// Decode attention in bfloat16 with the scores on the tensor cores.  The kernels above spend
// most of their issue slots on the softmax of each key, repeated in every lane that shares
// the key; here the work of a tile is spread differently:
//   scores : S = Q K^T by mma.sync.m16n8k16.  The rows of the 16-row operand are the query
//            heads of this key/value head (RB <= 8 of them, the rest zero), the 8 columns are
//            8 keys of the staged tile.  Each thread reads 16 contiguous bytes of a key and
//            uses them for two k-steps; the query fragments are permuted the same way.
//   softmax: the 8 x RB scores of a warp sit one pair per lane, so cap, mask, max, exp run
//            once per score, not once per lane group.
//   values : every lane owns 8 features (16 bytes) of the head and adds p * v for each key of
//            its warp; p comes by shuffle from the lane that holds it.
// Staging (bulk copies, mbarriers, bounded waits), chunking and the merge are those of the
// staged kernel.  Needs a tile of 32 or 64 keys: head sizes up to 256.
// ---------------------------------------------------------------------------
// out[s, heads of head group `y`, :] = v   (a padding row: 0; a sequence the launch was not sized for: NaN)
__device__ __forceinline__ void fill_heads(bf16* out, int s, int nq, int nkv, int y, int rb, float v) {
    const int rep = nq / nkv;
    const int groups = (rep + rb - 1) / rb;
    const int kvh = y / groups, hg = y % groups;
    const int h0 = kvh * rep + hg * rb, nh = min(rb, rep - hg * rb);
    for (int idx = threadIdx.x; idx < nh * HD; idx += blockDim.x)
        out[((size_t)s * nq + h0 + idx / HD) * HD + idx % HD] = __float2bfloat16_rn(v);
}

// NS stages: three give a CTA a deeper pipeline, two leave room for three CTAs an SM instead of two.  With more CTAs
// than two an SM can hold, more CTAs in flight pay more than depth (64 sequences of unequal lengths: 63.6 -> 56.5 us a
// layer with two stages; 8 sequences of 8,100 keys: 49.5 -> 47.8 us); with fewer CTAs than that, depth does (one
// sequence: 523 against 545 tok/s); four stages and one CTA an SM are far slower (98 us).  The launch chooses.
// WIDE: stages of 64 keys at head sizes above 128 too (a warp then has two column tiles of scores in flight): for
// launches with no more CTAs than SMs, where a CTA has an SM's shared memory to itself and the time of a tile, not
// the CTAs an SM holds, sets the pace (one sequence: 2.7 us for a tile of 32 keys, a CTA's chunk of 64 keys 5.4 us).
template <int NS, bool WIDE = false>
struct MmaDecode {
    static constexpr int WARPS = 4;
    static constexpr int STAGES = NS;
    static constexpr int TILE = (HD <= 128 || WIDE) ? 64 : 32;       // keys per stage
    static constexpr int NT = TILE / 32;                              // 8-key column tiles per warp and stage
    static constexpr int TILE_BYTES = TILE * HD * 2;
    static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES;
    static constexpr int KB = (HD + 31) / 32;                         // blocks of 32 features
    static constexpr int CH = HD / 8;                                 // 16-byte pieces of a value row
    static constexpr int CHL = CH >= 32 ? 32 : pow2_ceil(CH);         // lanes set aside for a value row (a power of two)
    static constexpr int CPV = (CH + 31) / 32;                        // pieces per lane
    static constexpr int KPI = 32 / CHL;                              // keys per load instruction
    static constexpr bool OK = HD <= 256;
};

// DIRECT: the launch has one chunk per sequence and the kernel writes the result itself (`out`); otherwise it
// leaves a partial per chunk for the merge kernel.
template <int RB, bool DIRECT, int NS, bool WIDE = false>
__global__ void __launch_bounds__(MmaDecode<NS, WIDE>::WARPS * 32)
attn_decode_mma_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ kpool, const bf16* __restrict__ vpool,
                       const int* __restrict__ page_table, int table_stride, const int* __restrict__ seq_slot,
                       const int* __restrict__ seq_len, float* __restrict__ partial, int nq, int nkv, int q_row_heads,
                       float scale, float cap, int window, int ring_len, int chunk, bf16* __restrict__ out) {
    typedef MmaDecode<NS, WIDE> S;
    extern __shared__ __align__(128) unsigned char stage_mem[];
    __shared__ __align__(8) unsigned long long full[S::STAGES];
    const int s = blockIdx.z;
    grid_dependents_launch();
    // The step's tables (slots, lengths, pages) are written before the step's first kernel, and every
    // key but the newest was stored by an earlier step: the first tiles are asked for before this
    // kernel waits for the one that stores the newest key and rotates the queries.
    const int slot = seq_slot[s];
    const int len = seq_len[s];                      // (asked for together: one trip to memory, not two)
    if (slot < 0) {
        grid_dependency_wait();
        if (DIRECT) fill_heads(out, s, nq, nkv, blockIdx.y, RB, 0.f);   // a padding row
        return;
    }
    int lo, first_chunk, n_chunks;
    chunk_range(len, window, chunk, lo, first_chunk, n_chunks);
    if (DIRECT && n_chunks > 1) {
        // the launch was sized for shorter sequences: make it visible, as the merge kernel does
        grid_dependency_wait();
        fill_heads(out, s, nq, nkv, blockIdx.y, RB, __int_as_float(0x7fc00000));
        return;
    }
    if ((int)blockIdx.x >= n_chunks) { grid_dependency_wait(); return; }
    const int c = first_chunk + blockIdx.x;
    const int k_begin = max(lo, c * chunk), k_end = min(len, (c + 1) * chunk);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int rep = nq / nkv;
    const int groups = (rep + RB - 1) / RB;
    const int kvh = blockIdx.y / groups, hg = blockIdx.y % groups;
    const int h0 = kvh * rep + hg * RB;
    const int nh_here = min(RB, rep - hg * RB);

    const uint32_t stage0 = (uint32_t)__cvta_generic_to_shared(stage_mem);
    const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(full);
    if (threadIdx.x == 0) {
        for (int i = 0; i < S::STAGES; ++i) mbar_init(bar0 + 8 * i, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();
    const int t_first = (k_begin / S::TILE) * S::TILE;
    const int n_tiles = (k_end - t_first + S::TILE - 1) / S::TILE;
    const int* table = page_table + (size_t)slot * table_stride;
    auto page_of = [&](int i) {                      // the page that holds tile i
        const int p0 = t_first + i * S::TILE;
        return table[(ring_len > 0 ? p0 % ring_len : p0) / JANIS_PAGE];
    };
    auto issue_from = [&](int i, int page) {
        const int p0 = t_first + i * S::TILE;
        const int idx = ring_len > 0 ? p0 % ring_len : p0;
        const size_t off = (((size_t)page * nkv + kvh) * JANIS_PAGE + idx % JANIS_PAGE) * HD;
        const int st_i = i % S::STAGES;
        const uint32_t dst = stage0 + st_i * S::STAGE_BYTES, bar = bar0 + 8 * st_i;
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        mbar_expect_tx(bar, S::STAGE_BYTES);
        bulk_load(dst, kpool + off, S::TILE_BYTES, bar);
        bulk_load(dst + S::TILE_BYTES, vpool + off, S::TILE_BYTES, bar);
    };
    auto issue = [&](int i) {
        const int p0 = t_first + i * S::TILE;
        const int idx = ring_len > 0 ? p0 % ring_len : p0;
        const int page = table[idx / JANIS_PAGE];
        const size_t off = (((size_t)page * nkv + kvh) * JANIS_PAGE + idx % JANIS_PAGE) * HD;
        const int st_i = i % S::STAGES;
        const uint32_t dst = stage0 + st_i * S::STAGE_BYTES, bar = bar0 + 8 * st_i;
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        mbar_expect_tx(bar, S::STAGE_BYTES);
        bulk_load(dst, kpool + off, S::TILE_BYTES, bar);
        bulk_load(dst + S::TILE_BYTES, vpool + off, S::TILE_BYTES, bar);
    };
    // a tile may be read early unless it holds the place the newest key goes to (position len - 1, which
    // in a ring is also the place of position len - 1 - ring_len)
    auto early = [&](int i) {
        const int p0 = t_first + i * S::TILE;
        const int newest = len - 1, shadow = len - 1 - ring_len;
        return !(newest >= p0 && newest < p0 + S::TILE) && !(ring_len > 0 && shadow >= p0 && shadow < p0 + S::TILE);
    };
    int first_pages[S::STAGES];                      // asked for together, before any of them is needed
    if (threadIdx.x == 0) {
#pragma unroll
        for (int i = 0; i < S::STAGES; ++i) first_pages[i] = i < n_tiles ? page_of(i) : 0;
#pragma unroll
        for (int i = 0; i < S::STAGES; ++i)
            if (i < n_tiles && early(i)) issue_from(i, first_pages[i]);
    }
    grid_dependency_wait();
    if (threadIdx.x == 0) {
#pragma unroll
        for (int i = 0; i < S::STAGES; ++i)
            if (i < n_tiles && !early(i)) issue_from(i, first_pages[i]);
    }

    // query fragments: row g of the 16-row operand is head h0 + g (zero beyond nh_here); a thread keeps, for
    // each block of 32 features, the 8 features t*8 .. t*8+7 as the pairs that two k-steps want
    uint32_t qf[S::KB][4];
    {
        const bf16* qrow = qkv + (size_t)s * q_row_heads * HD + (size_t)(h0 + g) * HD;
#pragma unroll
        for (int kb = 0; kb < S::KB; ++kb) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (g < nh_here && kb * 32 + t * 8 < HD) v = *reinterpret_cast<const uint4*>(qrow + kb * 32 + t * 8);
            qf[kb][0] = v.x; qf[kb][1] = v.y; qf[kb][2] = v.z; qf[kb][3] = v.w;
        }
    }
    // values: lane -> (key within a load instruction, 16-byte piece)
    const int ksub = lane / S::CHL, piece = lane % S::CHL;
    float acc[RB][S::CPV * 8];
#pragma unroll
    for (int r = 0; r < RB; ++r)
#pragma unroll
        for (int e = 0; e < S::CPV * 8; ++e) acc[r][e] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;          // of row g, the same in the four lanes that share it
    const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;

    for (int i = 0; i < n_tiles; ++i) {
        const int st_i = i % S::STAGES;
        const bool landed = mbar_wait(bar0 + 8 * st_i, (i / S::STAGES) & 1);
        if (landed) {
            const unsigned char* ks = stage_mem + (size_t)st_i * S::STAGE_BYTES;
            const unsigned char* vs = ks + S::TILE_BYTES;
            const int kw = warp * 8 * S::NT;                     // this warp's first key in the tile
            const int p0 = t_first + i * S::TILE + kw;           // its position
            // ---- scores
            float sc[S::NT][2];
#pragma unroll
            for (int nt = 0; nt < S::NT; ++nt) {
                float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
                const unsigned char* krow = ks + (size_t)(kw + nt * 8 + g) * HD * 2 + t * 16;
#pragma unroll
                for (int kb = 0; kb < S::KB; ++kb) {
                    uint4 kv = make_uint4(0, 0, 0, 0);
                    if (kb * 32 + t * 8 < HD) kv = *reinterpret_cast<const uint4*>(krow + kb * 64);
                    mma_rows8(c0, qf[kb][0], qf[kb][1], kv.x, kv.y);
                    mma_rows8(c1, qf[kb][2], qf[kb][3], kv.z, kv.w);
                }
                sc[nt][0] = c0[0] + c1[0];
                sc[nt][1] = c0[1] + c1[1];
            }
            // ---- cap, mask, running maximum and sum of row g over this warp's keys
            float mx = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < S::NT; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int j = p0 + nt * 8 + t * 2 + e;
                    float v = sc[nt][e] * scale;
                    if (cap > 0.f) v = cap * tanhf(v * inv_cap);
                    v = (j >= k_begin && j < k_end && g < nh_here) ? v : -INFINITY;
                    sc[nt][e] = v;
                    mx = fmaxf(mx, v);
                }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run, mx);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            const float corr = expf(m_run - m_use);               // exp(-inf) = 0 the first time
            float psum = 0.f;
#pragma unroll
            for (int nt = 0; nt < S::NT; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    sc[nt][e] = expf(sc[nt][e] - m_use);          // now the weight p of (row g, key)
                    psum += sc[nt][e];
                }
            l_run = l_run * corr + psum;
            m_run = m_new;
            // ---- values: acc[r] = acc[r] * corr_r + sum over keys of p[r][key] * v[key]
#pragma unroll
            for (int r = 0; r < RB; ++r) {
                const float cr = __shfl_sync(0xffffffffu, corr, r * 4);
#pragma unroll
                for (int e = 0; e < S::CPV * 8; ++e) acc[r][e] *= cr;
            }
#pragma unroll
            for (int nt = 0; nt < S::NT; ++nt) {
#pragma unroll
                for (int j0 = 0; j0 < 8; j0 += S::KPI) {
                    const int jk = j0 + ksub;                      // key of this lane, 0..7 within the column tile
                    const int pos = p0 + nt * 8 + jk;
                    const bool use = ksub < S::KPI && jk < 8 && pos >= k_begin && pos < k_end;
                    float pw[RB];
#pragma unroll
                    for (int r = 0; r < RB; ++r) {               // p[r][jk] lives in lane r*4 + jk/2, register jk%2
                        const float pe = __shfl_sync(0xffffffffu, sc[nt][0], r * 4 + ((jk & 7) >> 1));
                        const float po = __shfl_sync(0xffffffffu, sc[nt][1], r * 4 + ((jk & 7) >> 1));
                        pw[r] = (jk & 1) ? po : pe;
                    }
                    if (use) {
#pragma unroll
                        for (int cp = 0; cp < S::CPV; ++cp) {
                            const int pc = piece + cp * 32;
                            if (pc < S::CH) {
                                float vf[8];
                                Vec16<bf16>::load(reinterpret_cast<const bf16*>(vs + (size_t)(kw + nt * 8 + jk) * HD * 2) + pc * 8, vf);
#pragma unroll
                                for (int r = 0; r < RB; ++r)
#pragma unroll
                                    for (int e = 0; e < 8; ++e) acc[r][cp * 8 + e] = fmaf(pw[r], vf[e], acc[r][cp * 8 + e]);
                            }
                        }
                    }
                }
            }
        }
        if (!__syncthreads_and(landed ? 1 : 0)) {
            if (threadIdx.x == 0) atomicAdd(&g_wait_timeouts, 1);
            return;
        }
        if (threadIdx.x == 0 && i + S::STAGES < n_tiles) issue(i + S::STAGES);
    }
    // ---- this warp's state into shared memory (the stages are free now), then the warps in order
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
#pragma unroll
    for (int o = S::CHL; o < 32; o <<= 1)                      // lanes that took different keys of a load
#pragma unroll
        for (int r = 0; r < RB; ++r)
#pragma unroll
            for (int e = 0; e < S::CPV * 8; ++e) acc[r][e] += __shfl_xor_sync(0xffffffffu, acc[r][e], o);
    static_assert(sizeof(float) * S::WARPS * RB * (HD + 2) <= S::SMEM_BYTES, "the merge does not fit the stages");
    float (*sm)[RB][HD + 2] = reinterpret_cast<float (*)[RB][HD + 2]>(stage_mem);
    if (t == 0 && g < RB) { sm[warp][g][0] = m_run; sm[warp][g][1] = l_run; }
    if (ksub == 0) {
#pragma unroll
        for (int r = 0; r < RB; ++r)
#pragma unroll
            for (int cp = 0; cp < S::CPV; ++cp) {
                const int pc = piece + cp * 32;
                if (pc < S::CH) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) sm[warp][r][2 + pc * 8 + e] = acc[r][cp * 8 + e];
                }
            }
    }
    __syncthreads();
    const int max_chunks = gridDim.x;
    // the warps' states in warp order
    if (DIRECT) {
        // one chunk per sequence: the result itself
        for (int idx = threadIdx.x; idx < nh_here * HD; idx += blockDim.x) {
            const int r = idx / HD, d = idx % HD;
            float mx = -INFINITY;
#pragma unroll
            for (int w = 0; w < S::WARPS; ++w) mx = fmaxf(mx, sm[w][r][0]);
            float v = 0.f, l = 0.f;
#pragma unroll
            for (int w = 0; w < S::WARPS; ++w) {
                const float mw = sm[w][r][0];
                if (mw != -INFINITY) {
                    const float e = expf(mw - mx);
                    v += sm[w][r][2 + d] * e;
                    l += sm[w][r][1] * e;
                }
            }
            out[((size_t)s * nq + h0 + r) * HD + d] = __float2bfloat16_rn(v / l);
        }
    } else {
        for (int idx = threadIdx.x; idx < nh_here * (HD + 2); idx += blockDim.x) {
            const int r = idx / (HD + 2), d = idx % (HD + 2);
            float mx = -INFINITY;
#pragma unroll
            for (int w = 0; w < S::WARPS; ++w) mx = fmaxf(mx, sm[w][r][0]);
            float v;
            if (d == 0) v = mx;
            else {
                v = 0.f;
#pragma unroll
                for (int w = 0; w < S::WARPS; ++w) {
                    const float mw = sm[w][r][0];
                    if (mw != -INFINITY) v += sm[w][r][d] * expf(mw - mx);
                }
            }
            partial[(((size_t)s * nq + h0 + r) * max_chunks + blockIdx.x) * (HD + 2) + d] = v;
        }
    }
}

// Merge of the chunks in ascending order.  One CTA per (sequence, head): the chunks' weights
// exp(m_c - m) / l are formed once in shared memory, then each thread sums its features.
template <typename T>
__global__ void attn_merge_kernel(const float* __restrict__ partial, const int* __restrict__ seq_slot,
                                  const int* __restrict__ seq_len, T* __restrict__ out, int nq, int max_chunks,
                                  int window, int chunk) {
    extern __shared__ float wgt[];            // max_chunks weights
    __shared__ float red[32];
    const int s = blockIdx.x, h = blockIdx.y;
    grid_dependents_launch();
    const int slot = seq_slot[s], len = seq_len[s];          // the step's tables: read before the wait
    grid_dependency_wait();
    T* o = out + ((size_t)s * nq + h) * HD;
    if (slot < 0) {
        for (int d = threadIdx.x; d < HD; d += blockDim.x) o[d] = from_float<T>(0.f);
        return;
    }
    int lo, first_chunk, n_chunks;
    chunk_range(len, window, chunk, lo, first_chunk, n_chunks);
    if (n_chunks > max_chunks) {   // the launch was sized for shorter sequences: make it visible
        for (int d = threadIdx.x; d < HD; d += blockDim.x) o[d] = from_float<T>(__int_as_float(0x7fc00000));
        return;
    }
    const float* p = partial + ((size_t)s * nq + h) * max_chunks * (HD + 2);
    const int lane = threadIdx.x & 31;
    if (n_chunks <= 32) {
        // Up to 32 chunks: every warp forms the weights by itself, lane c for chunk c, and hands them round by
        // shuffles: one trip to memory for the maxima and sums, one for the values, no block barrier.
        const bool mine = lane < n_chunks;
        const float mc = mine ? p[(size_t)lane * (HD + 2)] : -INFINITY;
        const float lc = mine ? p[(size_t)lane * (HD + 2) + 1] : 0.f;
        const float mx = warp_max(mc);
        const float w = mc == -INFINITY ? 0.f : expf(mc - mx);
        float l = 0.f;                           // in chunk order, the same in every thread
        for (int c = 0; c < n_chunks; ++c) l += __shfl_sync(0xffffffffu, lc * w, c);
        const float inv = 1.0f / l;
        for (int d0 = 0; d0 < HD; d0 += blockDim.x) {         // the same trips for every lane: the shuffles stay whole
            const int d = d0 + threadIdx.x;
            float a0 = 0.f, a1 = 0.f;
            int c = 0;
            for (; c + 2 <= n_chunks; c += 2) {
                const float w0 = __shfl_sync(0xffffffffu, w, c), w1 = __shfl_sync(0xffffffffu, w, c + 1);
                if (d < HD) {
                    a0 += p[(size_t)c * (HD + 2) + 2 + d] * w0;
                    a1 += p[(size_t)(c + 1) * (HD + 2) + 2 + d] * w1;
                }
            }
            if (c < n_chunks) {
                const float w0 = __shfl_sync(0xffffffffu, w, c);
                if (d < HD) a0 += p[(size_t)c * (HD + 2) + 2 + d] * w0;
            }
            if (d < HD) o[d] = from_float<T>((a0 + a1) * inv);
        }
        return;
    }
    if (n_chunks <= 64) {
        // 33 to 64 chunks: the same with two chunks a lane (c and c + 32), still without a block barrier
        const bool m0 = lane < n_chunks, m1 = lane + 32 < n_chunks;
        const float mc0 = m0 ? p[(size_t)lane * (HD + 2)] : -INFINITY;
        const float lc0 = m0 ? p[(size_t)lane * (HD + 2) + 1] : 0.f;
        const float mc1 = m1 ? p[(size_t)(lane + 32) * (HD + 2)] : -INFINITY;
        const float lc1 = m1 ? p[(size_t)(lane + 32) * (HD + 2) + 1] : 0.f;
        const float mx = warp_max(fmaxf(mc0, mc1));
        const float w_lo = mc0 == -INFINITY ? 0.f : expf(mc0 - mx), w_hi = mc1 == -INFINITY ? 0.f : expf(mc1 - mx);
        float l = 0.f;                           // in chunk order, the same in every thread
        for (int c = 0; c < 32; ++c) l += __shfl_sync(0xffffffffu, lc0 * w_lo, c);
        for (int c = 32; c < n_chunks; ++c) l += __shfl_sync(0xffffffffu, lc1 * w_hi, c - 32);
        const float inv = 1.0f / l;
        for (int d0 = 0; d0 < HD; d0 += blockDim.x) {
            const int d = d0 + threadIdx.x;
            float a0 = 0.f, a1 = 0.f;
            int c = 0;
            for (; c + 2 <= n_chunks; c += 2) {          // (c is even: c and c + 1 lie in the same half)
                const float w0 = __shfl_sync(0xffffffffu, c < 32 ? w_lo : w_hi, c & 31);
                const float w1 = __shfl_sync(0xffffffffu, c < 32 ? w_lo : w_hi, (c + 1) & 31);
                if (d < HD) {
                    a0 += p[(size_t)c * (HD + 2) + 2 + d] * w0;
                    a1 += p[(size_t)(c + 1) * (HD + 2) + 2 + d] * w1;
                }
            }
            if (c < n_chunks) {
                const float w0 = __shfl_sync(0xffffffffu, c < 32 ? w_lo : w_hi, c & 31);
                if (d < HD) a0 += p[(size_t)c * (HD + 2) + 2 + d] * w0;
            }
            if (d < HD) o[d] = from_float<T>((a0 + a1) * inv);
        }
        return;
    }
    // the maximum over chunks (any order gives the same value)
    float mx = -INFINITY;
    for (int c = threadIdx.x; c < n_chunks; c += blockDim.x) mx = fmaxf(mx, p[(size_t)c * (HD + 2)]);
    mx = warp_max(mx);
    if (lane == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = red[0];
    for (int w = 1; w < (int)((blockDim.x + 31) >> 5); ++w) mx = fmaxf(mx, red[w]);
    for (int c = threadIdx.x; c < n_chunks; c += blockDim.x) {
        const float mc = p[(size_t)c * (HD + 2)];
        wgt[c] = mc == -INFINITY ? 0.f : expf(mc - mx);
    }
    __syncthreads();
    float l = 0.f;                               // in chunk order, the same in every thread
    for (int c = 0; c < n_chunks; ++c) l += p[(size_t)c * (HD + 2) + 1] * wgt[c];
    const float inv = 1.0f / l;
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;     // four running sums keep four loads in flight
        int c = 0;
        for (; c + 4 <= n_chunks; c += 4) {
            a0 += p[(size_t)(c + 0) * (HD + 2) + 2 + d] * wgt[c + 0];
            a1 += p[(size_t)(c + 1) * (HD + 2) + 2 + d] * wgt[c + 1];
            a2 += p[(size_t)(c + 2) * (HD + 2) + 2 + d] * wgt[c + 2];
            a3 += p[(size_t)(c + 3) * (HD + 2) + 2 + d] * wgt[c + 3];
        }
        for (; c < n_chunks; ++c) a0 += p[(size_t)c * (HD + 2) + 2 + d] * wgt[c];
        o[d] = from_float<T>(((a0 + a1) + (a2 + a3)) * inv);
    }
}

}  // namespace janis

using namespace janis;

JANIS_EXPORT int janis_attn_head_dim() { return HD; }

// 0: launch every kernel of this library plainly; 1 (default): let a kernel's CTAs arrive while the one before it runs
JANIS_EXPORT void janis_attn_set_overlap(int on) { overlap_launches() = on ? 1 : 0; }

// floats of scratch that a decode call with these sizes needs
JANIS_EXPORT long long janis_attn_decode_scratch(int n_seq, int nq, int max_chunks) {
    return (long long)n_seq * nq * max_chunks * (HD + 2);
}

// qkv: [T, q_row_heads, hd] holds the queries in its first nq heads; keys and values of position j of a
// sequence are read from row (seq_first_row + j) of kv_src, a [rows, kv_row_heads, hd]
// buffer whose key heads start at head kv_k_head0 and value heads nkv later
// (kv_src = qkv, kv_row_heads = nq + 2 nkv, kv_k_head0 = nq for a layer's own keys).
// With seq_start (int32 [n_seq], tokens of each sequence that earlier steps stored) the step continues sequences:
// seq_first_row is then the row of a sequence's first token of this step, and the keys and values of positions
// below seq_start come from the cache line (kpool, vpool, page_table, ring_len as in janis_attn_decode).
JANIS_EXPORT int janis_attn_prefill(const void* qkv, const void* kv_src, int dtype, const int* tok_pos,
                                    const int* tok_seq, const int* seq_first_row, void* out, int n_tok, int nq,
                                    int nkv, int q_row_heads, int kv_row_heads, int kv_k_head0, float scale,
                                    float cap, int window, const int* seq_start, const int* seq_slot,
                                    const void* kpool, const void* vpool, const int* page_table, int table_stride,
                                    int ring_len, cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    if (nkv <= 0 || nq % nkv) return fail("attn_prefill: %d query heads do not divide over %d key heads", nq, nkv);
    if (seq_start != nullptr && (seq_slot == nullptr || kpool == nullptr || vpool == nullptr || page_table == nullptr))
        return fail("attn_prefill: sequences that continue need their slots and the cache line");
    if (ring_len % JANIS_PAGE) return fail("attn_prefill: ring length %d is not a multiple of the page", ring_len);
    const CachedPrefix cached = {seq_start, seq_slot, kpool, vpool, page_table, table_stride, ring_len};
    const int rep = nq / nkv;
    dim3 grid((n_tok + ATTN_WARPS - 1) / ATTN_WARPS, 1, 1);
    if (dtype == JANIS_F32) {
        grid.y = nkv * ((rep + Geo<float>::RG - 1) / Geo<float>::RG);
        return launch_kernel("attn_prefill", attn_prefill_kernel<float>, grid, dim3(ATTN_WARPS * 32), 0, stream, 1,
                             (const float*)qkv, (const float*)kv_src, tok_pos, tok_seq, seq_first_row, (float*)out, n_tok, nq,
                             nkv, q_row_heads, kv_row_heads, kv_k_head0, scale, cap, window, cached);
    }
    if (dtype == JANIS_BF16) {
        grid.y = nkv * ((rep + Geo<bf16>::RG - 1) / Geo<bf16>::RG);
        return launch_kernel("attn_prefill", attn_prefill_kernel<bf16>, grid, dim3(ATTN_WARPS * 32), 0, stream, 1,
                             (const bf16*)qkv, (const bf16*)kv_src, tok_pos, tok_seq, seq_first_row, (bf16*)out, n_tok, nq,
                             nkv, q_row_heads, kv_row_heads, kv_k_head0, scale, cap, window, cached);
    }
    return fail("attn_prefill: unknown dtype %d", dtype);
}

static int g_decode_kernel = 2;     // 2: staged, scores on the tensor cores (bfloat16, head sizes <= 256);
                                    // 1: staged, CUDA cores; 0: straight from global memory into registers

// Which decode kernel janis_attn_decode launches (both give the same results up to rounding).
JANIS_EXPORT void janis_attn_set_decode_kernel(int which) { g_decode_kernel = which < 0 ? 0 : (which > 2 ? 2 : which); }

// How often a decode CTA has given up waiting for its bulk copies since the library was loaded
// (0 unless something is badly wrong).  Synchronises the device.
JANIS_EXPORT int janis_attn_wait_timeouts() {
    int n = -1;
    if (cudaMemcpyFromSymbol(&n, g_wait_timeouts, sizeof(int)) != cudaSuccess) return -1;
    return n;
}

namespace janis { int prefill_tc05_timeouts_async(int* host, cudaStream_t stream); }   // attention_prefill_tc05.cu

// Both counts of this library (host[0]: the decode kernels' waits, host[1]: the tcgen05 prompt kernel's) copied into
// pinned host memory in the order of `stream`, without waiting for it: a caller that waits for the stream anyway
// (for its tokens) finds them there afterwards.
JANIS_EXPORT int janis_attn_timeouts_async(int* host, cudaStream_t stream) {
    cudaError_t e = cudaMemcpyFromSymbolAsync(host, g_wait_timeouts, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
    if (e != cudaSuccess) return fail("attn_timeouts_async: %s", cudaGetErrorString(e));
    return prefill_tc05_timeouts_async(host + 1, stream);
}

// Runs the bounded wait against a barrier nothing completes (at most 4096 tries): *status becomes 1.
JANIS_EXPORT int janis_attn_wait_probe(int tries, int* status, cudaStream_t stream) {
    if (tries < 1 || tries > 4096) return fail("wait_probe: between 1 and 4096 tries, found %d", tries);
    wait_probe_kernel<<<1, 32, 0, stream>>>(tries, status);
    return launched("wait_probe");
}

template <int RB, int NS, bool WIDE = false>
static int launch_decode_mma_ns(const bf16* qkv, const bf16* kpool, const bf16* vpool, const int* page_table,
                                int table_stride, const int* seq_slot, const int* seq_len, float* partial, int n_seq, int nq,
                                int nkv, int q_row_heads, float scale, float cap, int window, int ring_len, int chunk,
                                int max_chunks, bf16* out, cudaStream_t stream) {
    typedef MmaDecode<NS, WIDE> S;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_mma_kernel<RB, false, NS, WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             S::SMEM_BYTES);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(attn_decode_mma_kernel<RB, true, NS, WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     S::SMEM_BYTES);
        if (e != cudaSuccess) return fail("attn_decode: shared memory of %d bytes refused: %s", S::SMEM_BYTES,
                                          cudaGetErrorString(e));
        configured = true;
    }
    const int rep = nq / nkv;
    dim3 grid(max_chunks, nkv * ((rep + RB - 1) / RB), n_seq);
    if (out != nullptr)
        return launch_kernel("attn_decode", attn_decode_mma_kernel<RB, true, NS, WIDE>, grid, dim3(S::WARPS * 32),
                             S::SMEM_BYTES, stream, 1, qkv, kpool, vpool, page_table, table_stride, seq_slot, seq_len,
                             partial, nq, nkv, q_row_heads, scale, cap, window, ring_len, chunk, out);
    return launch_kernel("attn_decode", attn_decode_mma_kernel<RB, false, NS, WIDE>, grid, dim3(S::WARPS * 32),
                         S::SMEM_BYTES, stream, 1, qkv, kpool, vpool, page_table, table_stride, seq_slot, seq_len,
                         partial, nq, nkv, q_row_heads, scale, cap, window, ring_len, chunk, out);
}

static int decode_sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
    }
    return n;
}

static int g_mma_wide = 1;          // 0: never the stages of 64 keys at head sizes above 128 (tests and tuning)
JANIS_EXPORT void janis_attn_set_decode_wide(int on) { g_mma_wide = on ? 1 : 0; }

static int g_mma_stages = 0;        // 0: chosen per launch from the number of CTAs; 2 or 3: fixed (tests and tuning)

// Fixes the stages of the tensor-core decode kernel (2 or 3; 0: chosen from the launch's size again).
JANIS_EXPORT void janis_attn_set_decode_stages(int stages) { g_mma_stages = stages == 2 || stages == 3 ? stages : 0; }

// How many stages a launch of this many CTAs gets: two (three CTAs an SM) when it has more CTAs than two an SM would
// hold at once, else three.  The host sizes its chunks by the same rule.
JANIS_EXPORT int janis_attn_decode_stages(long long n_ctas) {
    if (g_mma_stages) return g_mma_stages;
    return n_ctas > 2LL * decode_sm_count() ? 2 : 3;
}

template <int RB>
static int launch_decode_mma_rb(const bf16* qkv, const bf16* kpool, const bf16* vpool, const int* page_table,
                                int table_stride, const int* seq_slot, const int* seq_len, float* partial, int n_seq, int nq,
                                int nkv, int q_row_heads, float scale, float cap, int window, int ring_len, int chunk,
                                int max_chunks, bf16* out, cudaStream_t stream) {
    const int rep = nq / nkv;
    const long long n_ctas = (long long)max_chunks * nkv * ((rep + RB - 1) / RB) * n_seq;
    if (HD > 128 && g_mma_wide && n_ctas <= decode_sm_count())       // a CTA an SM at most: stages of 64 keys
        return launch_decode_mma_ns<RB, 2, true>(qkv, kpool, vpool, page_table, table_stride, seq_slot, seq_len, partial, n_seq, nq,
                                                 nkv, q_row_heads, scale, cap, window, ring_len, chunk, max_chunks, out, stream);
    if (janis_attn_decode_stages(n_ctas) == 2)
        return launch_decode_mma_ns<RB, 2>(qkv, kpool, vpool, page_table, table_stride, seq_slot, seq_len, partial, n_seq, nq, nkv,
                                           q_row_heads, scale, cap, window, ring_len, chunk, max_chunks, out, stream);
    return launch_decode_mma_ns<RB, 3>(qkv, kpool, vpool, page_table, table_stride, seq_slot, seq_len, partial, n_seq, nq, nkv,
                                       q_row_heads, scale, cap, window, ring_len, chunk, max_chunks, out, stream);
}

static int launch_decode_mma(const bf16* qkv, const bf16* kpool, const bf16* vpool, const int* page_table, int table_stride,
                             const int* seq_slot, const int* seq_len, float* partial, int n_seq, int nq, int nkv,
                             int q_row_heads, float scale, float cap, int window, int ring_len, int chunk, int max_chunks,
                             bf16* out, cudaStream_t stream) {
    const int rep = nq / nkv;
#define JANIS_RB(RB)                                                                                                   \
    return launch_decode_mma_rb<RB>(qkv, kpool, vpool, page_table, table_stride, seq_slot, seq_len, partial, n_seq, nq, nkv, \
                                    q_row_heads, scale, cap, window, ring_len, chunk, max_chunks, out, stream)
    if (rep == 1) JANIS_RB(1);
    if (rep == 2) JANIS_RB(2);
    if (rep <= 4) JANIS_RB(4);
    JANIS_RB(8);
#undef JANIS_RB
}

template <typename T>
static int launch_decode(const T* qkv, const T* kpool, const T* vpool, const int* page_table, int table_stride,
                         const int* seq_slot, const int* seq_len, float* partial, T* out, int n_seq, int nq, int nkv,
                         int q_row_heads, float scale, float cap, int window, int ring_len, int chunk, int max_chunks,
                         cudaStream_t stream) {
    const int rep = nq / nkv;
    if (g_decode_kernel == 2 && sizeof(T) == 2 && MmaDecode<2>::OK) {
        // a launch of one chunk per sequence writes the result itself: no partials, no merge
        bf16* direct = max_chunks == 1 ? (bf16*)out : nullptr;
        if (launch_decode_mma((const bf16*)qkv, (const bf16*)kpool, (const bf16*)vpool, page_table, table_stride, seq_slot,
                              seq_len, partial, n_seq, nq, nkv, q_row_heads, scale, cap, window, ring_len, chunk, max_chunks,
                              direct, stream))
            return 1;
        if (direct != nullptr) return 0;
    } else if (g_decode_kernel >= 1) {
        typedef Geo<T, Staged<T>::LMAX, Staged<T>::BUDGET> GS;
        dim3 grid(max_chunks, nkv * ((rep + GS::RG - 1) / GS::RG), n_seq);
        static bool configured = false;
        if (!configured) {
            cudaError_t e = cudaFuncSetAttribute(attn_decode_staged_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 Staged<T>::SMEM_BYTES);
            if (e != cudaSuccess) return fail("attn_decode: shared memory of %d bytes refused: %s", Staged<T>::SMEM_BYTES,
                                              cudaGetErrorString(e));
            configured = true;
        }
        if (launch_kernel("attn_decode", attn_decode_staged_kernel<T>, grid, dim3(Staged<T>::WARPS * 32), Staged<T>::SMEM_BYTES,
                          stream, 1, qkv, kpool, vpool, page_table, table_stride, seq_slot, seq_len, partial, nq, nkv,
                          q_row_heads, scale, cap, window, ring_len, chunk))
            return 1;
    } else {
        dim3 grid(max_chunks, nkv * ((rep + Geo<T>::RG - 1) / Geo<T>::RG), n_seq);
        if (launch_kernel("attn_decode", attn_decode_kernel<T>, grid, dim3(ATTN_WARPS * 32), 0, stream, 1, qkv, kpool, vpool,
                          page_table, table_stride, seq_slot, seq_len, partial, nq, nkv, q_row_heads, scale, cap, window,
                          ring_len, chunk))
            return 1;
    }
    dim3 mgrid(n_seq, nq);
    const int mthreads = HD < 256 ? (HD < 32 ? 32 : HD) : 256;
    return launch_kernel("attn_merge", attn_merge_kernel<T>, mgrid, dim3(mthreads), max_chunks * sizeof(float), stream, 1,
                         (const float*)partial, seq_slot, seq_len, out, nq, max_chunks, window, chunk);
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
    if (max_chunks > 8192) return fail("attn_decode: too many chunks (%d)", max_chunks);
    if (dtype == JANIS_F32)
        return launch_decode<float>((const float*)qkv, (const float*)kpool, (const float*)vpool, page_table, table_stride,
                                    seq_slot, seq_len, partial, (float*)out, n_seq, nq, nkv, q_row_heads, scale, cap,
                                    window, ring_len, chunk, max_chunks, stream);
    if (dtype == JANIS_BF16)
        return launch_decode<bf16>((const bf16*)qkv, (const bf16*)kpool, (const bf16*)vpool, page_table, table_stride,
                                   seq_slot, seq_len, partial, (bf16*)out, n_seq, nq, nkv, q_row_heads, scale, cap,
                                   window, ring_len, chunk, max_chunks, stream);
    return fail("attn_decode: unknown dtype %d", dtype);
}

JANIS_EXPORT const char* janis_last_error() { return error_buffer(); }
