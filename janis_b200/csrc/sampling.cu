// Choosing the next token from float logits [R, V] on the device: greedy (the
// lowest id among equal maxima), temperature with an optional nucleus (top-p)
// cut, the repetition penalty, and masking of given ids.  One CTA per row; all
// sums run in a fixed order, so a row's choice depends on the row alone.
//
// The random number of a draw is Philox4x32-10 keyed by the seed and counted by
// (request id, index of the token in its reply): it does not depend on which
// other requests share the batch.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace janis {

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
    const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
    const uint32_t hi0 = __umulhi(M0, c[0]), lo0 = M0 * c[0];
    const uint32_t hi1 = __umulhi(M1, c[2]), lo1 = M1 * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

__device__ __forceinline__ float philox_uniform(unsigned long long seed, uint32_t request, uint32_t index) {
    uint32_t c[4] = {request, index, 0u, 0u};
    uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        philox_round(c, k0, k1);
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return (float)(c[0] >> 8) * (1.0f / 16777216.0f);   // [0, 1), 24 bits
}

// max of a row with the lowest index that attains it; every thread gets both
__device__ void block_argmax(float v, int i, float* sv, int* si, float& out_v, int& out_i) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
    __syncthreads();
    if (lane == 0) { sv[warp] = v; si[warp] = i; }
    __syncthreads();
    float bv = sv[0];
    int bi = si[0];
    for (int w = 1; w < nwarp; ++w)
        if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
    out_v = bv;
    out_i = bi;
}

// The largest value of row[lo, hi) and the lowest id that attains it, as far as this thread's ids go (they
// ascend, so `>` keeps the lowest).  Four independent loads per round keep the memory pipe busy.
__device__ __forceinline__ void argmax_scan(const float* __restrict__ row, int lo, int hi, float& v, int& i) {
    int j = lo + threadIdx.x;
    if ((lo & 3) == 0 && (((uintptr_t)row) & 15) == 0) {
        // 16-byte loads, two in flight per round; within a load the ids ascend, across rounds too
        const float4* row4 = reinterpret_cast<const float4*>(row);
        const int q_end = lo / 4 + (hi - lo) / 4;
        int q = lo / 4 + threadIdx.x;
        for (; q + (int)blockDim.x < q_end; q += 2 * blockDim.x) {
            const float4 a = row4[q], b = row4[q + blockDim.x];
            const int ja = q * 4, jb = (q + blockDim.x) * 4;
            if (a.x > v) { v = a.x; i = ja; }
            if (a.y > v) { v = a.y; i = ja + 1; }
            if (a.z > v) { v = a.z; i = ja + 2; }
            if (a.w > v) { v = a.w; i = ja + 3; }
            if (b.x > v) { v = b.x; i = jb; }
            if (b.y > v) { v = b.y; i = jb + 1; }
            if (b.z > v) { v = b.z; i = jb + 2; }
            if (b.w > v) { v = b.w; i = jb + 3; }
        }
        for (; q < q_end; q += blockDim.x) {
            const float4 a = row4[q];
            const int ja = q * 4;
            if (a.x > v) { v = a.x; i = ja; }
            if (a.y > v) { v = a.y; i = ja + 1; }
            if (a.z > v) { v = a.z; i = ja + 2; }
            if (a.w > v) { v = a.w; i = ja + 3; }
        }
        j = q_end * 4 + threadIdx.x;                       // the few ids the 16-byte loads left over
    }
    for (; j + 3 * (int)blockDim.x < hi; j += 4 * blockDim.x) {
        const float x0 = row[j], x1 = row[j + blockDim.x], x2 = row[j + 2 * blockDim.x], x3 = row[j + 3 * blockDim.x];
        if (x0 > v) { v = x0; i = j; }                       // NaN never wins
        if (x1 > v) { v = x1; i = j + blockDim.x; }
        if (x2 > v) { v = x2; i = j + 2 * blockDim.x; }
        if (x3 > v) { v = x3; i = j + 3 * blockDim.x; }
    }
    for (; j < hi; j += blockDim.x) {
        const float x = row[j];
        if (x > v) { v = x; i = j; }
    }
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int V) {
    __shared__ float sv[32];
    __shared__ int si[32];
    const float* row = logits + (size_t)blockIdx.x * V;
    grid_dependents_launch();
    grid_dependency_wait();
    float v = -INFINITY;
    int i = 0x7fffffff;
    argmax_scan(row, 0, V, v, i);
    float bv;
    int bi;
    block_argmax(v, i, sv, si, bv, bi);
    if (threadIdx.x == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
}

// The same for few rows of a large vocabulary: a thread-block cluster of ARGMAX_CLUSTER CTAs shares a row,
// each takes a stretch of ids, and CTA 0 picks among their results through distributed shared memory
// (one CTA reads a row of 256,000 logits in 24 us; eight read it in 5).
constexpr int ARGMAX_CLUSTER = 8;

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_cluster_kernel(const float* __restrict__ logits, int* __restrict__ out, int V) {
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ float best_v;
    __shared__ int best_i;
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank(), r = blockIdx.x / ARGMAX_CLUSTER;
    const float* row = logits + (size_t)r * V;
    const int seg = ((V + ARGMAX_CLUSTER - 1) / ARGMAX_CLUSTER + 3) & ~3;      // a multiple of 4: stretches start 16-byte aligned
    const int lo = min(V, rank * seg), hi = min(V, lo + seg);
    grid_dependents_launch();
    grid_dependency_wait();
    float v = -INFINITY;
    int i = 0x7fffffff;
    argmax_scan(row, lo, hi, v, i);
    float bv;
    int bi;
    block_argmax(v, i, sv, si, bv, bi);
    if (threadIdx.x == 0) { best_v = bv; best_i = bi; }
    cluster.sync();                                  // every CTA's result is in its shared memory
    if (rank == 0 && threadIdx.x == 0) {
        for (int c = 1; c < ARGMAX_CLUSTER; ++c) {   // stretches ascend with the rank: `>` keeps the lowest id
            const float ov = *cluster.map_shared_rank(&best_v, c);
            const int oi = *cluster.map_shared_rank(&best_i, c);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        out[r] = bi == 0x7fffffff ? 0 : bi;
    }
    cluster.sync();                                  // nobody leaves while its shared memory is being read
}

// Exclusive scan of one value per thread, in thread order, by thread 0.
__device__ float block_exclusive_scan(float v, float* buf, float& total) {
    __syncthreads();
    buf[threadIdx.x] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        float run = 0.f;
        for (int i = 0; i < (int)blockDim.x; ++i) {
            const float x = buf[i];
            buf[i] = run;
            run += x;
        }
        buf[blockDim.x] = run;
    }
    __syncthreads();
    total = buf[blockDim.x];
    return buf[threadIdx.x];
}

// Temperature sampling of one row.  w_j = exp((l_j - max) / temp).  With top_p < 1
// the kept set is the shortest prefix, in descending w with ties to the lower id,
// whose mass reaches top_p of the total; the draw is the inverse CDF over the kept
// ids in id order at r = u * kept mass.  Thread i owns the contiguous ids
// [i * per, (i + 1) * per), so thread order is id order.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int* __restrict__ out, float* __restrict__ u_out, int V,
              float temp, float top_p, unsigned long long seed, const int* __restrict__ request_ids,
              const int* __restrict__ token_index) {
    __shared__ float buf[SAMPLE_THREADS + 1];
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ int chosen;
    grid_dependents_launch();
    grid_dependency_wait();
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * V;
    const int per = (V + blockDim.x - 1) / blockDim.x;
    const int lo = min((int)threadIdx.x * per, V), hi = min(lo + per, V);

    float v = -INFINITY;
    int vi = 0x7fffffff;
    for (int j = threadIdx.x; j < V; j += blockDim.x) {
        const float x = row[j];
        if (x > v || (x == v && j < vi)) { v = x; vi = j; }
    }
    float mx;
    int mi;
    block_argmax(v, vi, sv, si, mx, mi);
    const float inv_t = 1.0f / temp;

    float total;
    float mine = 0.f;
    for (int j = lo; j < hi; ++j) mine += expf((row[j] - mx) * inv_t);
    block_exclusive_scan(mine, buf, total);

    // nucleus: the largest threshold tau with mass(w >= tau) >= top_p * total
    float tau = 0.f;
    int ties_kept = 0x7fffffff;
    const bool cut = top_p > 0.f && top_p < 1.f;
    if (cut) {
        const float need = top_p * total;
        uint32_t blo = 0u, bhi = __float_as_uint(1.0f);   // w lies in [0, 1]; mass(w >= 0) = total >= need
        while (blo < bhi) {                               // invariant: mass(w >= blo) >= need
            const uint32_t mid = blo + (bhi - blo + 1) / 2;
            const float th = __uint_as_float(mid);
            float m = 0.f;
            for (int j = lo; j < hi; ++j) {
                const float w = expf((row[j] - mx) * inv_t);
                if (w >= th) m += w;
            }
            float mass;
            block_exclusive_scan(m, buf, mass);
            if (mass >= need) blo = mid; else bhi = mid - 1;
        }
        tau = __uint_as_float(blo);
        float above = 0.f;
        for (int j = lo; j < hi; ++j) {
            const float w = expf((row[j] - mx) * inv_t);
            if (w > tau) above += w;
        }
        float mass_above;
        block_exclusive_scan(above, buf, mass_above);
        // the fewest ties, lowest ids first, that lift the mass to `need`
        ties_kept = tau > 0.f ? (int)ceilf((need - mass_above) / tau) : 0x7fffffff;
        if (ties_kept < 1) ties_kept = 1;
    }

    // kept mass per thread, with the rank of each tie in id order
    float tie_count = 0.f;
    if (cut)
        for (int j = lo; j < hi; ++j) tie_count += (expf((row[j] - mx) * inv_t) == tau) ? 1.f : 0.f;
    float tie_total;
    const float tie_before = cut ? block_exclusive_scan(tie_count, buf, tie_total) : 0.f;
    float kept = 0.f;
    {
        int rank = (int)tie_before;
        for (int j = lo; j < hi; ++j) {
            const float w = expf((row[j] - mx) * inv_t);
            bool keep = true;
            if (cut) {
                if (w == tau) { keep = rank < ties_kept; ++rank; }
                else keep = w > tau;
            }
            if (keep) kept += w;
        }
    }
    float kept_total;
    const float before = block_exclusive_scan(kept, buf, kept_total);

    const float u = philox_uniform(seed, (uint32_t)request_ids[r], (uint32_t)token_index[r]);
    const float target = u * kept_total;
    if (threadIdx.x == 0) {
        chosen = 0x7fffffff;
        if (u_out) u_out[r] = u;
    }
    __syncthreads();
    // the owner of the target walks its ids; `before <= target` holds for thread 0 always
    if (kept > 0.f && before <= target && target <= before + kept) {
        int rank = (int)tie_before;
        float acc = before;
        int pick = -1, last = -1;
        for (int j = lo; j < hi; ++j) {
            const float w = expf((row[j] - mx) * inv_t);
            bool keep = true;
            if (cut) {
                if (w == tau) { keep = rank < ties_kept; ++rank; }
                else keep = w > tau;
            }
            if (!keep) continue;
            acc += w;
            last = j;
            if (target <= acc) { pick = j; break; }
        }
        if (pick < 0) pick = last;
        if (pick >= 0) atomicMin(&chosen, pick);   // see below
    }
    __syncthreads();
    // Two neighbouring threads can both claim a target that sits on their border;
    // the lower id is the inverse CDF's answer, so take the minimum of the claims.
    if (threadIdx.x == 0) out[r] = chosen != 0x7fffffff ? chosen : mi;
}

__global__ void repeat_penalty_kernel(float* __restrict__ logits, const int* __restrict__ recent, int n_recent,
                                      int V, float penalty) {
    // recent: [R, n_recent], -1 where empty.  A token that occurs twice is changed once.
    const int r = blockIdx.x;
    grid_dependents_launch();
    grid_dependency_wait();
    const int* rec = recent + (size_t)r * n_recent;
    for (int i = threadIdx.x; i < n_recent; i += blockDim.x) {
        const int tok = rec[i];
        if (tok < 0 || tok >= V) continue;
        bool first = true;
        for (int j = 0; j < i; ++j)
            if (rec[j] == tok) { first = false; break; }
        if (!first) continue;
        float* p = logits + (size_t)r * V + tok;
        const float v = *p;
        *p = v > 0.f ? v / penalty : v * penalty;
    }
}

__global__ void mask_tokens_kernel(float* __restrict__ logits, const int* __restrict__ ids, int n_ids, int R,
                                   int V) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    grid_dependents_launch();
    grid_dependency_wait();
    if (idx >= R * n_ids) return;
    const int r = idx / n_ids, tok = ids[idx % n_ids];
    if (tok >= 0 && tok < V) logits[(size_t)r * V + tok] = -INFINITY;
}

}  // namespace janis

using namespace janis;

JANIS_EXPORT int janis_argmax(const float* logits, int* out, int R, int V, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0) return fail("argmax: empty vocabulary");
    if (R <= 32 && V >= 16384)
        return launch_kernel("argmax", argmax_cluster_kernel, dim3(R * ARGMAX_CLUSTER), dim3(SAMPLE_THREADS), 0, stream,
                             ARGMAX_CLUSTER, logits, out, V);
    return launch_kernel("argmax", argmax_kernel, dim3(R), dim3(SAMPLE_THREADS), 0, stream, 1, logits, out, V);
}

// ---------------------------------------------------------------------------
// The same choice with the row's weights held in shared memory.  The kernel above reads its row from global
// memory once per pass (some thirty-five passes with a nucleus, each thread walking a stretch of its own, which a
// warp's loads do not coalesce) and scans in one thread: 1.9 ms for 8 rows of 256,000 logits.  Here a thread-block
// cluster of CL CTAs shares a row: each CTA computes the weights of its stretch once (coalesced loads), keeps them
// in shared memory, and every later pass reads shared memory only; a thread owns `per` consecutive ids (an odd
// number: no bank conflicts), so thread order within a CTA and CTA order within the cluster are id order.  Sums
// over threads are prefix sums by shuffles in a fixed tree, sums over CTAs are added in CTA order from slots that
// every CTA fills in all the others' shared memory; every CTA sees the same numbers and takes the same branches.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float block_prefix(float v, float* wtot, float& total) {
    // exclusive prefix of v in thread order and the block's total; wtot: 33 floats of shared memory
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    float incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    float excl = __shfl_up_sync(0xffffffffu, incl, 1);
    if (lane == 0) excl = 0.f;
    __syncthreads();                                  // wtot may still be read from the call before
    if (lane == 31) wtot[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const float t = lane < nwarp ? wtot[lane] : 0.f;
        float ti = t;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, ti, o);
            if (lane >= o) ti += up;
        }
        float te = __shfl_up_sync(0xffffffffu, ti, 1);
        if (lane == 0) te = 0.f;
        const float all = __shfl_sync(0xffffffffu, ti, 31);
        wtot[lane] = te;
        if (lane == 0) wtot[32] = all;
    }
    __syncthreads();
    total = wtot[32];
    return wtot[warp] + excl;
}

template <int CL> struct ClusterSlots {
    float f[2][CL];                                    // two sets, used in turn: a CTA fills set k + 2 only after every
    int i[2][CL];                                      // CTA has passed the barrier of set k + 1, i.e. has read set k
};

// every CTA's value, in CTA order: returns the sum of the CTAs before this one and the sum of all
template <int CL>
__device__ __forceinline__ float cluster_prefix(float mine, ClusterSlots<CL>* slots, int& turn, int rank, float& total) {
    if (CL == 1) { total = mine; return 0.f; }
    cg::cluster_group cluster = cg::this_cluster();
    const int set = turn & 1;
    ++turn;
    if (threadIdx.x < CL) cluster.map_shared_rank(slots, threadIdx.x)->f[set][rank] = mine;
    cluster.sync();
    float before = 0.f, run = 0.f;
#pragma unroll
    for (int c = 0; c < CL; ++c) {
        if (c == rank) before = run;
        run += slots->f[set][c];
    }
    total = run;
    return before;
}

template <int CL>
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_shared_kernel(const float* __restrict__ logits, int* __restrict__ out, float* __restrict__ u_out, int V,
                     float temp, float top_p, unsigned long long seed, const int* __restrict__ request_ids,
                     const int* __restrict__ token_index, int seg, int per) {
    extern __shared__ float w[];                      // this CTA's stretch of weights: per * SAMPLE_THREADS floats
    __shared__ float wtot[33];
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ ClusterSlots<CL> slots;
    __shared__ int chosen;
    const int rank = CL == 1 ? 0 : (int)cg::this_cluster().block_rank();
    const int r = blockIdx.x / CL;
    const float* row = logits + (size_t)r * V;
    const int base = min(V, rank * seg), n_here = min(V, base + seg) - base;      // ids [base, base + n_here)
    const int lo = min((int)threadIdx.x * per, n_here), hi = min(lo + per, n_here); // this thread's, within the stretch
    int turn = 0;
    grid_dependents_launch();
    if (CL > 1) cg::this_cluster().sync();            // a CTA's shared memory may be written by the others once it runs
    grid_dependency_wait();

    // the row's maximum and the lowest id that attains it
    float v = -INFINITY;
    int vi = 0x7fffffff;
    for (int j = threadIdx.x; j < n_here; j += blockDim.x) {
        const float x = row[base + j];
        if (x > v) { v = x; vi = base + j; }            // ids ascend within a thread: `>` keeps the lowest
    }
    float mx;
    int mi;
    block_argmax(v, vi, sv, si, mx, mi);
    if (CL > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        if (threadIdx.x < CL) {
            ClusterSlots<CL>* remote = cluster.map_shared_rank(&slots, threadIdx.x);
            remote->f[0][rank] = mx;
            remote->i[0][rank] = mi;
        }
        ++turn;
        cluster.sync();
        mx = slots.f[0][0];
        mi = slots.i[0][0];
#pragma unroll
        for (int c = 1; c < CL; ++c)
            if (slots.f[0][c] > mx || (slots.f[0][c] == mx && slots.i[0][c] < mi)) { mx = slots.f[0][c]; mi = slots.i[0][c]; }
    }
    const float inv_t = 1.0f / temp;
    for (int j = threadIdx.x; j < n_here; j += blockDim.x) w[j] = expf((row[base + j] - mx) * inv_t);
    __syncthreads();

    float mine = 0.f, here, total;
    for (int j = lo; j < hi; ++j) mine += w[j];
    block_prefix(mine, wtot, here);
    cluster_prefix<CL>(here, &slots, turn, rank, total);

    // nucleus: the largest threshold tau with mass(w >= tau) >= top_p * total
    float tau = 0.f;
    int ties_kept = 0x7fffffff;
    const bool cut = top_p > 0.f && top_p < 1.f;
    if (cut) {
        const float need = top_p * total;
        uint32_t blo = 0u, bhi = __float_as_uint(1.0f);   // w lies in [0, 1]; mass(w >= 0) = total >= need
        while (blo < bhi) {                               // invariant: mass(w >= blo) >= need
            const uint32_t mid = blo + (bhi - blo + 1) / 2;
            const float th = __uint_as_float(mid);
            float m = 0.f;
            for (int j = lo; j < hi; ++j) {
                const float x = w[j];
                if (x >= th) m += x;
            }
            float m_here, mass;
            block_prefix(m, wtot, m_here);
            cluster_prefix<CL>(m_here, &slots, turn, rank, mass);
            if (mass >= need) blo = mid; else bhi = mid - 1;
        }
        tau = __uint_as_float(blo);
        float above = 0.f;
        for (int j = lo; j < hi; ++j) {
            const float x = w[j];
            if (x > tau) above += x;
        }
        float above_here, mass_above;
        block_prefix(above, wtot, above_here);
        cluster_prefix<CL>(above_here, &slots, turn, rank, mass_above);
        // the fewest ties, lowest ids first, that lift the mass to `need`
        ties_kept = tau > 0.f ? (int)ceilf((need - mass_above) / tau) : 0x7fffffff;
        if (ties_kept < 1) ties_kept = 1;
    }

    // kept mass per thread, with the rank of each tie in id order
    float tie_before = 0.f;
    if (cut) {
        float tie_count = 0.f, ties_here, ties_all;
        for (int j = lo; j < hi; ++j) tie_count += (w[j] == tau) ? 1.f : 0.f;
        tie_before = block_prefix(tie_count, wtot, ties_here);
        tie_before += cluster_prefix<CL>(ties_here, &slots, turn, rank, ties_all);
    }
    float kept = 0.f;
    {
        int tie_rank = (int)tie_before;
        for (int j = lo; j < hi; ++j) {
            const float x = w[j];
            bool keep = true;
            if (cut) {
                if (x == tau) { keep = tie_rank < ties_kept; ++tie_rank; }
                else keep = x > tau;
            }
            if (keep) kept += x;
        }
    }
    float kept_here, kept_total;
    float before = block_prefix(kept, wtot, kept_here);
    before += cluster_prefix<CL>(kept_here, &slots, turn, rank, kept_total);

    const float u = philox_uniform(seed, (uint32_t)request_ids[r], (uint32_t)token_index[r]);
    const float target = u * kept_total;
    if (threadIdx.x == 0) {
        chosen = 0x7fffffff;
        if (u_out && rank == 0) u_out[r] = u;
    }
    __syncthreads();
    // the owner of the target walks its ids; two neighbours can both claim a target that sits on their border:
    // the lower id is the inverse CDF's answer, so the minimum of the claims is taken
    if (kept > 0.f && before <= target && target <= before + kept) {
        int tie_rank = (int)tie_before;
        float acc = before;
        int pick = -1, last = -1;
        for (int j = lo; j < hi; ++j) {
            const float x = w[j];
            bool keep = true;
            if (cut) {
                if (x == tau) { keep = tie_rank < ties_kept; ++tie_rank; }
                else keep = x > tau;
            }
            if (!keep) continue;
            acc += x;
            last = base + j;
            if (target <= acc) { pick = base + j; break; }
        }
        if (pick < 0) pick = last;
        if (pick >= 0) atomicMin(&chosen, pick);
    }
    __syncthreads();
    int best = chosen;
    if (CL > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        const int set = turn & 1;
        if (threadIdx.x < CL) cluster.map_shared_rank(&slots, threadIdx.x)->i[set][rank] = best;
        cluster.sync();
#pragma unroll
        for (int c = 0; c < CL; ++c) best = min(best, slots.i[set][c]);
        cluster.sync();                               // nobody leaves while its shared memory may still be written
    }
    if (rank == 0 && threadIdx.x == 0) out[r] = best != 0x7fffffff ? best : mi;
}

template <int CL>
static int launch_sample_shared(const float* logits, int* out, float* u_out, int R, int V, float temp, float top_p,
                                unsigned long long seed, const int* request_ids, const int* token_index, cudaStream_t stream) {
    const int seg = ((V + CL - 1) / CL + 3) & ~3;
    int per = (seg + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    per |= 1;                                          // odd: threads that walk their stretches hit different banks
    const size_t smem = (size_t)per * SAMPLE_THREADS * sizeof(float);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(sample_shared_kernel<CL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return fail("sample: shared memory refused: %s", cudaGetErrorString(e));
        configured = true;
    }
    return launch_kernel("sample", sample_shared_kernel<CL>, dim3(R * CL), dim3(SAMPLE_THREADS), smem, stream, CL, logits, out,
                         u_out, V, temp, top_p, seed, request_ids, token_index, seg, per);
}

static int g_sample_kernel = 1;     // 1: weights in shared memory where the vocabulary fits a cluster's; 0: the global-memory kernel

// Which kernel janis_sample launches (for tests: both make the same choice up to the rounding of their sums).
JANIS_EXPORT void janis_set_sample_kernel(int which) { g_sample_kernel = which ? 1 : 0; }

JANIS_EXPORT int janis_sample(const float* logits, int* out, float* u_out, int R, int V, float temp, float top_p,
                              unsigned long long seed, const int* request_ids, const int* token_index,
                              cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0) return fail("sample: empty vocabulary");
    if (!(temp > 0.f)) return fail("sample: temperature must be positive (greedy is argmax), found %g", temp);
    if (g_sample_kernel == 1) {
        const int fits = 45 * SAMPLE_THREADS;          // floats of shared memory a CTA gives to its stretch (180 KB)
#define JANIS_SAMPLE(CL) \
    return launch_sample_shared<CL>(logits, out, u_out, R, V, temp, top_p, seed, request_ids, token_index, stream)
        if (V <= fits) JANIS_SAMPLE(1);
        if (V <= 2 * fits - 8) JANIS_SAMPLE(2);
        if (V <= 4 * fits - 16) JANIS_SAMPLE(4);
        if (V <= 8 * fits - 32) JANIS_SAMPLE(8);
#undef JANIS_SAMPLE
    }
    return launch_kernel("sample", sample_kernel, dim3(R), dim3(SAMPLE_THREADS), 0, stream, 1, logits, out, u_out, V, temp,
                         top_p, seed, request_ids, token_index);
}

JANIS_EXPORT int janis_repeat_penalty(float* logits, const int* recent, int n_recent, int R, int V, float penalty,
                                      cudaStream_t stream) {
    if (R <= 0 || n_recent <= 0 || !(penalty > 1.f)) return 0;
    return launch_kernel("repeat_penalty", repeat_penalty_kernel, dim3(R), dim3(64), 0, stream, 1, logits, recent, n_recent,
                         V, penalty);
}

JANIS_EXPORT int janis_mask_tokens(float* logits, const int* ids, int n_ids, int R, int V, cudaStream_t stream) {
    if (R <= 0 || n_ids <= 0) return 0;
    const int n = R * n_ids;
    return launch_kernel("mask_tokens", mask_tokens_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, 1, logits, ids,
                         n_ids, R, V);
}
