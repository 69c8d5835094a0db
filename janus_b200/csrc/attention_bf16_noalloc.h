// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (DaCodeChick/Janus
// allocates all of its buffers up front through wgpu); it exists for users of
// this library whose code runs where cudaMalloc is off limits: inside another
// framework's memory plan, in a process whose whole device budget was handed
// out at start-up, or on a latency path where an allocator call may block.
//
// It runs the same split-key decode attention as jb_attention_bf16_decode, but
// the partial results of the key splits (float32 partial outputs, maxima and
// sums) live in a fixed array inside the library instead of a caller-provided
// scratch buffer.  Inputs and outputs are still the caller's.
//
//  * The array holds JB_NOALLOC_SCRATCH_FLOATS floats (4 MiB).  Every GPU that
//    loads this library keeps it until the process exits.  The attention
//    library is built once per head size (-DJB_HEAD_DIM), and each build is a
//    shared library of its own with an array of its own: a process that loads
//    the builds for four head sizes holds four arrays, 16 MiB per GPU.
//  * A call with n_splits > 1 needs n_seqs * n_heads * n_splits * (head_dim + 2)
//    floats; a call that needs more is refused with JB_ERR_BAD_SIZE and a
//    message on stderr.  With n_splits == 1 the kernel writes straight to
//    `out`, the array is not touched and any batch size is taken.
//  * The first call on a device looks up the array's device address
//    (cudaGetSymbolAddress, with that device current) and remembers it; make
//    that first call before any stream capture begins.  Several host threads
//    may make it at the same time.
//  * No cudaMalloc, cudaFree or allocating library routine is called, on the
//    first call or later.
//  * All calls share the one array, and it keeps the last call's contents.
//    Nothing in it has to start at zero: every entry that a launch reads was
//    written by the same launch.  Two calls that overlap on the GPU (different
//    streams, or graphs run side by side) race on it; keep calls on one
//    stream, or order them with events.
#pragma once
#include <cuda_runtime.h>

#define JB_NOALLOC_SCRATCH_FLOATS (1u << 20)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments as jb_attention_bf16_decode, without the two scratch pointers.
// Returns 0, a cudaError_t value, or a JB_ERR_* code.
int jb_attention_bf16_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                     const int* block_table, const int* kv_len, int n_seqs, int nh, int nkv,
                                     int hd, int page_size, int max_pages, int window, float scale,
                                     int n_splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
