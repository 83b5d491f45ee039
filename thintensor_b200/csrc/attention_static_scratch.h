// Split-key decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in random-unknown-username/Thintensor; it is this
// library's own addition.
//
// Who it is for.  tt_attention() (attention.cu) needs two scratch arrays for the partial
// results of the key slices, and leaves it to the caller to provide them; the Python
// package takes them from torch's allocator.  Some callers have no allocator to ask: a
// host program that links this library through its C interface alone and has already
// divided the GPU's memory between weights and cache at start-up, so that any later
// cudaMalloc could fail or fragment what it planned; a step that runs under a latency
// bound and may not pay for cudaMalloc's implicit device synchronisation; code that
// runs where only pre-registered buffers may be touched.  For them this entry point does
// the same computation with the scratch in an array that is part of the library's own
// image: nothing is allocated at any time, by any route.
//
// The price.  The array has a fixed size, TT_STATIC_SCRATCH_BYTES (16 MiB); every GPU on
// which this library is loaded holds that much from load until the process exits, used
// or not.  A call that needs more is refused (see the return values).  All calls share
// the one array, which still holds the previous call's partial results when the next
// call starts: nothing in it has to start at zero, because every (row, slice) entry is
// written by the first kernel before the second reads it, but two calls that overlap on
// the GPU (different streams, or two host threads) race on it and both give wrong
// results.  Issue calls one after another on one stream, or order them with events.
//
// Set-up.  The first call on each device looks up the array's device address
// (cudaGetSymbolAddress, with that device current) and keeps it; later calls on that
// device reuse it.  Because that lookup may initialise the library's image on the
// device, make the first call on a device before beginning any stream capture.
#pragma once
#include <cuda_runtime.h>

#define TT_STATIC_SCRATCH_BYTES (16u * 1024u * 1024u)

// Return values of tt_attention_decode_static besides cudaError_t values (> 0):
#define TT_STATIC_OK 0
#define TT_STATIC_TOO_LARGE (-1)   // the call needs more scratch than TT_STATIC_SCRATCH_BYTES
#define TT_STATIC_BAD_SIZE (-2)    // head size, head counts or splits the kernels do not take
#define TT_STATIC_NO_SYMBOL (-3)   // the array's address could not be obtained on this device

#ifdef __cplusplus
extern "C" {
#endif

// One query token per sequence (or any packed tokens) attending over the block cache,
// keys cut into `splits` slices.  Arguments are those of tt_attention() without the two
// scratch pointers.  Returns TT_STATIC_OK when both kernels were launched on `stream`.
int tt_attention_decode_static(const void* q, const void* k_pool, const void* v_pool, int dtype, const int* table,
                               int table_width, int pool_blocks, const int* cu, const int* len_before, int sequences,
                               int n_tokens, int heads, int kv_heads, int head_dim, float scale, int window,
                               int splits, void* out, unsigned* status, cudaStream_t stream);

// Bytes of scratch a call with these sizes needs; compare with TT_STATIC_SCRATCH_BYTES.
unsigned long long tt_attention_static_bytes_needed(int n_tokens, int heads, int head_dim, int splits);

// A sentence describing the last non-zero return value of this thread's calls.
const char* tt_attention_static_last_error(void);

#ifdef __cplusplus
}
#endif
