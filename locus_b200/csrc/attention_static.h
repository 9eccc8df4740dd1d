// Decode attention for callers that must not allocate.  This entry point has no counterpart
// in the reference (garana/locus); it exists for the users of this library described below.
//
// Who needs it.  The regular entry point, locus_attn_decode, wants two scratch buffers from
// its caller for the per-split partial results.  Some callers have no way to provide them:
// code that runs inside a region where device allocation is forbidden or would deadlock (a
// callback on a stream, a section that holds an allocator lock, a host that was given a
// fixed memory budget at start-up and no allocator handle at all), and plain C callers that
// link the library without a tensor library to allocate through.  For them the scratch lives
// inside the library, in a file-scope device array of fixed size.
//
// What it costs.  Every GPU on which the library is loaded holds
// LOCUS_ATTN_STATIC_SCRATCH_FLOATS * 4 bytes (4 MiB) for that array, and 64 KiB of counters, until the process ends,
// whether this entry point is ever called or not.
//
// Limit.  A call needs  n_items * n_heads * max_splits * (head_dim + 2)  floats of scratch and
// n_items * n_heads  counters.  Calls that need more than LOCUS_ATTN_STATIC_SCRATCH_FLOATS
// floats or LOCUS_ATTN_STATIC_COUNTERS counters are refused with LOCUS_ERR_SCRATCH_TOO_SMALL
// before anything is launched; use locus_attn_decode with buffers of your own for those.
//
// Rules of use.
//  * The first call on each device looks up the array's device address
//    (cudaGetSymbolAddress) with that device current.  Make that first call outside of any
//    stream capture.
//  * All calls share the one array, and it keeps whatever the last call left in it.  Nothing
//    in it has to start at zero: a call writes every element before it reads it.  The
//    counters (a second, small array) are zero when the library is loaded and every call
//    that completes leaves them zero.  Because the arrays are shared, two calls whose
//    kernels can overlap on the GPU (different streams, or different host threads) race;
//    order them on one stream or with events.
//  * max_splits must cover the longest context of the batch (longest position / 128 + 1).  The context
//    lengths live on the device, so the host cannot check this; a kernel that finds a longer context
//    reads only the keys that its splits cover, sets the module's error word (locus_attn_error()
//    returns 1 and clears it; the read synchronises) and still leaves the counters zero, so later
//    calls are not affected.  The output of that call is incomplete and must be discarded.
//  * It calls no cudaMalloc / cudaFree and no allocating library routine; inputs and outputs
//    are the caller's.
#pragma once

#include <cuda_runtime.h>

#define LOCUS_ATTN_STATIC_SCRATCH_FLOATS (1 << 20)
#define LOCUS_ATTN_STATIC_COUNTERS (1 << 14)
#define LOCUS_ERR_SCRATCH_TOO_SMALL 10002

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and results as locus_attn_decode, without part_o / part_ml (max_splits must
// cover the longest context: at least longest position / 128 + 1).
// Returns 0, a cudaError_t, LOCUS_ERR_UNSUPPORTED (10001) or LOCUS_ERR_SCRATCH_TOO_SMALL.
int locus_attn_decode_static(const void* q, int dt, const void* pool, void* out, const int* seg_q0,
                             const int* seg_qn, const int* seg_ctx, const int* block_table,
                             int table_stride, const int* items, int n_items, int nh, int nkv, int hd,
                             int page_tokens, int window, float scale, int max_splits,
                             cudaStream_t stream);

// 0, or the code that a kernel of this module recorded since the last call (then cleared).
int locus_attn_error(void);

#ifdef __cplusplus
}
#endif
