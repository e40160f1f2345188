// Shared helpers of the sm_100a kernels: error reporting to the host wrapper,
// conversions between storage types and float, 16-byte vector loads, and
// fixed-order reductions.  Every kernel computes in float whatever it stores.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#define JANIS_EXPORT extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python wrapper
#define JANIS_F32 0
#define JANIS_BF16 1

// tokens per cache page
#define JANIS_PAGE 64

namespace janis {

typedef __nv_bfloat16 bf16;

// One message per calling thread; the entry point that failed returns non-zero
// and the wrapper reads the text through janis_last_error().
inline char* error_buffer() {
    static thread_local char buf[512];
    return buf;
}

inline int fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return 1;
}

inline int launched(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail("%s: launch failed: %s", what, cudaGetErrorString(e));
    return 0;
}

// Programmatic dependent launch.  Every kernel of this library is launched so that
// its CTAs may become resident while the kernel before it in the stream is still
// running: it calls grid_dependents_launch() at its top and grid_dependency_wait()
// before it touches anything an earlier kernel wrote or still reads; one of the two
// (see JANIS_RUN_AHEAD) tells the hardware that the next kernel may start arriving.  What comes before the wait may only read constants of the
// model (weights).  The wait returns when the whole preceding grid has finished and
// its writes are visible, so the order of the stream is kept link by link.  Without
// the launch attribute both instructions do nothing.
//
// JANIS_RUN_AHEAD = 0 (default): the next kernel may arrive only once this one has passed its own
// wait, so at most two kernels share the GPU (one running, one with its weights on the way).
// JANIS_RUN_AHEAD = 1: the next kernel may arrive as soon as this one is resident, and so on down
// the stream; kernels that only wait then hold registers and shared memory of several layers.
#ifndef JANIS_RUN_AHEAD
#define JANIS_RUN_AHEAD 0
#endif
__device__ __forceinline__ void grid_dependency_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
#if !JANIS_RUN_AHEAD
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
}
__device__ __forceinline__ void grid_dependents_launch() {
#if JANIS_RUN_AHEAD
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
}

// The rotation of a rotary pair (a, b) by the angle whose sine and cosine are (s, c), with the roundings spelled
// out: left to the compiler, a * c - b * s contracts to one of two fused forms that differ in the last bit, and
// the kernels that rotate (the encoding kernels, the fused decode projection) must agree bit for bit.
__device__ __forceinline__ void rotate_pair(float a, float b, float s, float c, float& lo, float& hi) {
    lo = __fmaf_rn(a, c, -__fmul_rn(b, s));
    hi = __fmaf_rn(a, s, __fmul_rn(b, c));
}

// one switch per library (the wrapper sets it in each): 0 launches plainly
inline int& overlap_launches() {
    static int on = 1;
    return on;
}

// Launch with the attribute above, and as thread-block clusters of `cluster` CTAs when cluster > 1.
template <typename... KArgs, typename... Args>
inline int launch_kernel(const char* what, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                         cudaStream_t stream, int cluster, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (cluster > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    if (overlap_launches()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (e != cudaSuccess) return fail("%s: launch failed: %s", what, cudaGetErrorString(e));
    return 0;
}

// Where a multi-token step finds the keys and values of positions that earlier steps stored: the paged cache line
// ([pages, kv heads, JANIS_PAGE, head size]; position p of a sequence in page table[slot][p / JANIS_PAGE], or at
// p % ring_len for a windowed line).  seq_start == nullptr: every sequence of the step starts at position 0 and
// nothing is read from the cache.
struct CachedPrefix {
    const int* seq_start;      // [n_seq] tokens of each sequence stored before this step
    const int* seq_slot;       // [n_seq]
    const void* kpool;
    const void* vpool;
    const int* page_table;
    int table_stride;
    int ring_len;
};

__device__ __forceinline__ size_t cached_row(const CachedPrefix& c, int slot, int pos, int nkv, int kvh, int hd) {
    const int idx = c.ring_len > 0 ? pos % c.ring_len : pos;
    const int page = c.page_table[(size_t)slot * c.table_stride + idx / JANIS_PAGE];
    return (((size_t)page * nkv + kvh) * JANIS_PAGE + idx % JANIS_PAGE) * (size_t)hd;
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

// 16 bytes of T as floats
template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    __device__ __forceinline__ static void load(const float* p, float* out) {
        float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    }
    __device__ __forceinline__ static void store(float* p, const float* in) {
        *reinterpret_cast<float4*>(p) = make_float4(in[0], in[1], in[2], in[3]);
    }
};
template <> struct Vec16<bf16> {
    static constexpr int N = 8;
    __device__ __forceinline__ static void load(const bf16* p, float* out) {
        uint4 v = *reinterpret_cast<const uint4*>(p);
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {   // a bfloat16 is the upper half of a float
            out[2 * i] = __uint_as_float(w[i] << 16);
            out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    __device__ __forceinline__ static void store(bf16* p, const float* in) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block in a fixed order (warp butterflies, then warps in index
// order), so that a row's result does not depend on anything but the row.
// `scratch` holds at least 32 floats; every thread gets the total.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();            // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = 0.f;
    for (int w = 0; w < nwarp; ++w) t += scratch[w];
    return t;
}

__device__ __forceinline__ float gelu_tanh(float v) {
    const float inner = 0.7978845608028654f * (v + 0.044715f * v * v * v);
    return 0.5f * v * (1.0f + tanhf(inner));
}

}  // namespace janis
