// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference: there every tensor, scratch
// included, comes from the backend's allocator.  It exists for two kinds of caller of
// this library's C symbols.  One reaches the kernels from another runtime (a C, C++ or
// Go host through its foreign-function interface) and has neither torch's allocator nor
// a pool of its own at hand.  The other is a serving loop that has handed all device
// memory to the weights and the cache when it started: a cudaMalloc inside a step could
// fail there, and it would stall the device while it runs.  Both still own the tensors
// they pass in and get back; what they lack is a place for the kernel's scratch.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define JANIS_API __attribute__((visibility("default")))

// Floats of scratch held inside the library for janis_attn_decode_static: 2 Mi floats,
// 8 MiB.  The array is part of the image of one attention library, and there is one such
// library per head size: a process that loads the libraries of several head sizes holds
// 8 MiB for each of them, on every GPU on which it calls this entry point, until it exits
// (and calls through different libraries neither share an array nor race on one).
// When the memory is taken: the CUDA runtime loads a library's device code lazily, so the
// 8 MiB of a GPU are committed by the first call of janis_attn_decode_static on that GPU
// (its look-up of the array's address), not when the library is opened.  A caller that is
// about to give the rest of the device's memory away makes that first call before it does
// (a call with n_seq = 0 does the set-up and launches nothing); otherwise the first call
// may fail for lack of memory.  Later calls commit nothing more.
#define JANIS_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)

// The existing entry point: the caller passes `partial`, a float scratch of at least
// janis_attn_decode_scratch(n_seq, nq, max_chunks) floats.
JANIS_API int janis_attn_decode(const void* qkv, const void* kpool, const void* vpool, int dtype, const int* page_table,
                      int table_stride, const int* seq_slot, const int* seq_len, float* partial,
                      long long partial_floats, void* out, int n_seq, int nq, int nkv, int q_row_heads,
                      float scale, float cap, int window, int ring_len, int chunk, int max_chunks,
                      cudaStream_t stream);

JANIS_API long long janis_attn_decode_scratch(int n_seq, int nq, int max_chunks);

// The same computation with the same arguments, minus the scratch: it lives in a static
// device array of JANIS_STATIC_SCRATCH_FLOATS floats inside the library.  It calls no
// cudaMalloc, cudaFree or any routine that allocates; the caller passes inputs and outputs
// as before.
//
//  * Sizes: n_seq * nq * max_chunks * (head size + 2) floats must fit the array; a larger
//    request is refused (returns non-zero, janis_last_error() says how much was asked and how
//    much there is) and nothing is launched.
//  * First call on a device: it looks up the array's device address (cudaGetSymbolAddress,
//    with that device current) and remembers it per device; this is also when the array's
//    memory is committed (see above).  Make this first call outside any stream capture and
//    before memory runs short; n_seq = 0 is accepted for it (the other arguments are then
//    not looked at).  Later calls only launch the kernels.
//  * The array is shared by every call and keeps what the last call left.  Nothing in it has
//    to start at zero: each call writes every partial result that it reads afterwards, and
//    reads no other.  Two calls whose kernels overlap on the GPU (different streams, or
//    different threads on one device) race on the array: order them on one stream.
//
// Returns 0 on success.
JANIS_API int janis_attn_decode_static(const void* qkv, const void* kpool, const void* vpool, int dtype,
                             const int* page_table, int table_stride, const int* seq_slot, const int* seq_len,
                             void* out, int n_seq, int nq, int nkv, int q_row_heads, float scale, float cap,
                             int window, int ring_len, int chunk, int max_chunks, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
