// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference project: it is an
// addition of this library.
//
// Who needs it: code that runs where cudaMalloc is off limits.  A plugin called
// from inside somebody else's stream capture, a real-time loop that must not
// take the allocator's lock, a host application that hands this library a fixed
// memory budget and forbids it to grow: none of them can give
// vx_paged_decode_attention the scratch buffer it asks for by allocating one at
// call time.  For them the scratch lives inside the library, in a file-scope
// device array of fixed size that every GPU loading the library holds until the
// process exits (VX_DECODE_STATIC_SCRATCH_FLOATS floats = 16 MiB).
//
// Contract:
//   * Same arguments and same results as vx_paged_decode_attention, minus the
//     scratch pointer.  Inputs and outputs are still the caller's.
//   * max_splits must bound the pieces of every request in the call:
//     ceil(ceil(keys / 16) / chunk_tiles) for the request with the most keys, one
//     more if there is a window.  The device cannot tell the host that it was too
//     small: a request with more pieces than that loses its last keys (the result
//     is wrong), though nothing outside the scratch is read or written.
//   * The kernels run in plain stream order after whatever the caller launched
//     before (no programmatic dependent launch), so the caller's previous kernel
//     may write any of the inputs.
//   * Allocates nothing: no cudaMalloc, cudaFree or allocating library call.
//   * requests * H * max_splits * (D + 2) must not exceed
//     VX_DECODE_STATIC_SCRATCH_FLOATS; otherwise nothing runs and the call
//     returns VX_ERR_LIMIT (-4).  vx_paged_decode_static_max_floats() reports
//     the limit.
//   * The first call on each device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current) and configures the
//     kernel (every block shape it may pick for later steps).  Make that first
//     call before any stream capture begins, and from one host thread.
//   * All calls share the one array, and it keeps whatever the previous call
//     left in it.  The kernels write every scratch element before reading it,
//     so nothing needs clearing; but two calls that overlap on the GPU (on
//     different streams, say) race on it.  Serialise them.
#pragma once
#include <cuda_runtime.h>

#define VX_DECODE_STATIC_SCRATCH_FLOATS (4 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

long long vx_paged_decode_static_max_floats(void);

int vx_paged_decode_attention_static(const void* q, int q_row_stride, const void* k_pool, const void* v_pool,
                                     const int* block_table, int max_blocks, const int* token_rows,
                                     const int* seq_of_token, const int* positions, int max_splits, void* out,
                                     int out_row_stride, float scale, int window, int requests, int H, int Hk,
                                     int D, int S, int chunk_tiles, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
