// Declaration of the one entry point of this library that allocates nothing.
// It has no counterpart in the reference (cryptomilk/Crane allocates through
// its tensor library everywhere); it exists for callers of this library.
//
// Who needs it: a host program that has handed the whole device to an arena of
// its own (any cudaMalloc made on its behalf would fail or eat into memory it
// has promised elsewhere), and a serving loop that must not stall, since
// cudaMalloc and cudaFree synchronise the device and so hold up every stream
// of the process.  Such callers own all inputs and outputs and cannot give
// this library room for its intermediate results either.
//
// What it is: the split-KV decode attention of attention_decode.cu, with the
// per-slice partial results (max, sum, unnormalised output) kept in an array
// that is part of the library image instead of in buffers the caller passes.
//
//  * The array is CRANE_NOALLOC_SCRATCH_FLOATS floats (4 MiB).  Every GPU that
//    loads the library holds it from load until the process exits.
//  * n_splits is 1..64 (anything else: CRANE_NOALLOC_BAD_ARGUMENT).
//  * A call needs n_entries * nq * n_splits * (d + 2) floats of it.  A call
//    that needs more is refused with CRANE_NOALLOC_TOO_LARGE and launches
//    nothing; crane_noalloc_strerror() says so in words.  n_splits == 1 needs
//    none of it.
//  * The first call on a device looks the array's device address up
//    (cudaGetSymbolAddress, with that device current) and remembers it per
//    device.  Make that first call before any stream capture is begun.
//  * All calls share the one array, which keeps what the last call left.
//    Nothing in it has to start at zero: a call writes every slot that it later
//    reads.  For the same reason two calls that overlap on the GPU (different
//    streams, no dependency between them) race on the array: order them.
//  * It calls no cudaMalloc, cudaFree or other allocating routine.
#pragma once
#include <cuda_runtime.h>

#define CRANE_NOALLOC_SCRATCH_FLOATS (1 << 20)
#define CRANE_NOALLOC_TOO_LARGE (-2)
#define CRANE_NOALLOC_BAD_ARGUMENT (-3)
#define CRANE_NOALLOC_NO_SYMBOL (-4)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and result as crane_paged_decode_attention, without its two
// scratch pointers.  Returns 0, a CUDA error code (> 0) of the launch, or one of
// the negative codes above.
int crane_paged_decode_attention_noalloc(const void* q, void* out, const void* k_pool,
                                         const void* v_pool, const int* cu_q, const int* kv_len,
                                         const int* block_table, int max_blocks, int num_pages,
                                         int page_size, int n_entries, int nq, int nkv, int d,
                                         int window, float scale, int n_splits, int* err,
                                         cudaStream_t stream);

// Words for a negative code of the function above.
const char* crane_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
