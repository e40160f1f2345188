// janis_attn_decode_static: decode attention whose scratch is a static device array inside
// this library, for callers that cannot allocate (see attention_no_alloc.h, which holds the
// contract).  No counterpart in the reference.
#include "attention_no_alloc.h"

#include <mutex>

#include "common.cuh"

namespace {

// The scratch itself.  In host code this name is only a stand-in for the device object: a
// kernel must be given the address that cudaGetSymbolAddress returns, never this name.
static __device__ __align__(256) float g_decode_scratch[JANIS_STATIC_SCRATCH_FLOATS];

constexpr int MAX_DEVICES = 64;
float* g_scratch_address[MAX_DEVICES];     // per device, looked up once
std::mutex g_setup_lock;

// The device address of the scratch on the current device; nullptr (with the error text set) on failure.
float* scratch_on_current_device() {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        janis::fail("attn_decode_static: cudaGetDevice failed: %s", cudaGetErrorString(e));
        return nullptr;
    }
    if (dev < 0 || dev >= MAX_DEVICES) {
        janis::fail("attn_decode_static: device %d is outside the %d this library keeps addresses for", dev, MAX_DEVICES);
        return nullptr;
    }
    std::lock_guard<std::mutex> guard(g_setup_lock);
    if (g_scratch_address[dev] == nullptr) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_decode_scratch);
        if (e != cudaSuccess || p == nullptr) {
            janis::fail("attn_decode_static: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
            return nullptr;
        }
        g_scratch_address[dev] = p;
    }
    return g_scratch_address[dev];
}

}  // namespace

extern "C" JANIS_API int janis_attn_decode_static(const void* qkv, const void* kpool, const void* vpool, int dtype,
                                                  const int* page_table, int table_stride, const int* seq_slot,
                                                  const int* seq_len, void* out, int n_seq, int nq, int nkv,
                                                  int q_row_heads, float scale, float cap, int window, int ring_len,
                                                  int chunk, int max_chunks, cudaStream_t stream) {
    if (n_seq < 0) return janis::fail("attn_decode_static: a negative number of sequences");
    if (n_seq == 0) return scratch_on_current_device() == nullptr ? 1 : 0;     // the set-up alone: nothing to launch
    if (nq <= 0 || max_chunks <= 0) return janis::fail("attn_decode_static: nq and max_chunks must be positive");
    const long long need = janis_attn_decode_scratch(n_seq, nq, max_chunks);
    if (need > (long long)JANIS_STATIC_SCRATCH_FLOATS)
        return janis::fail("attn_decode_static: %d sequences x %d heads x %d chunks need %lld floats of scratch, the "
                           "static scratch holds %lld; use janis_attn_decode with a scratch of your own",
                           n_seq, nq, max_chunks, need, (long long)JANIS_STATIC_SCRATCH_FLOATS);
    float* scratch = scratch_on_current_device();
    if (scratch == nullptr) return 1;
    // every partial that the merge kernel reads is written by the decode kernel of this same call,
    // so what an earlier call left in the array does not matter and nothing is cleared
    return janis_attn_decode(qkv, kpool, vpool, dtype, page_table, table_stride, seq_slot, seq_len, scratch,
                             (long long)JANIS_STATIC_SCRATCH_FLOATS, out, n_seq, nq, nkv, q_row_heads, scale, cap,
                             window, ring_len, chunk, max_chunks, stream);
}
