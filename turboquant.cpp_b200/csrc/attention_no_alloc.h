// tq_attention_split_static — split attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference (its attention runs on the CPU and keeps its
// score buffer inside the per-sequence state, src/engine/tq_transformer.c:197-206); it exists for
// one class of users of this library.
//
// Who needs it.  tq_attention_split takes a `partial` buffer of scratch from its caller, and callers
// normally get that buffer from an allocator at call time.  Some callers cannot: a host program that
// handed all device memory to its own pool at start-up and forbids cudaMalloc afterwards, a plug-in
// running inside such a program, or code on a path where an allocation (and the implicit
// synchronisation cudaMalloc/cudaFree can cause) is not acceptable.  For them this variant keeps the
// scratch inside the library: a file-scope `static __device__ __align__(256)` array of
// TQ_ATTENTION_STATIC_SCRATCH_FLOATS floats (8 MiB) for the ranges' partial states, and one of
// TQ_ATTENTION_STATIC_ROWS ints (64 KiB) for the tickets by which the last range of a row finds that it is
// the last.  Every GPU on which the library is loaded holds both arrays until the process exits, whether
// or not this entry point is ever called.
//
// Contract.
//  * Same arguments and same result as tq_attention_split, without `partial`.  Inputs and the output
//    are still the caller's.
//  * It calls no cudaMalloc, cudaFree or any allocating library routine.
//  * It needs T * nh * n_splits * (hd + 2) floats of scratch and at most T * nh tickets; if that exceeds
//    TQ_ATTENTION_STATIC_SCRATCH_FLOATS or TQ_ATTENTION_STATIC_ROWS it returns an error (see
//    tq_last_error) and launches nothing.
//  * The first call on a device looks up the arrays' device addresses (cudaGetSymbolAddress, with that
//    device current) and remembers them per device.  Make that first call before any stream capture.
//  * All calls on a device share the arrays, which keep whatever the last call left in them.  The
//    partial states need not start at zero: every one that is read is written first by the same call.
//    The tickets must be zero when a call starts: they are when the library is loaded, and the kernel
//    itself sets a row's ticket back to zero once the row's last range has taken it, so a call that
//    ran to its end leaves them zero for the next.  Two calls that overlap on the GPU (different
//    streams, no ordering between them) race on both arrays; order them.
#pragma once
#include <cuda_runtime.h>

#define TQ_ATTENTION_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define TQ_ATTENTION_STATIC_ROWS (16 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

int tq_attention_split_static(const void* q, const void* cache, int act_dtype, const int* positions,
                              const int* seq_of_token, const int* page_table, int table_stride, int page_size,
                              int window, float scale, int n_splits, void* out, int T_, int nh, int nkv, int hd,
                              cudaStream_t stream);

#ifdef __cplusplus
}
#endif
