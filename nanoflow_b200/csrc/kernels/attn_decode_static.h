// Allocation-free split-KV decode attention.
//
// This entry point has no counterpart in the reference.
//
// nfk_attn_decode (kernels.h) needs a caller-provided fp32 workspace when the KV sequence is split
// into chunks (chunk_pages > 0). Some callers have no way to provide one: an engine that has
// already handed every free byte of device memory to its KV pool, or a host that calls this
// library from a place where it must not allocate (a plug-in callback, a serving loop with a
// no-allocation rule after start-up). For them nfk_attn_decode_static runs the same kernels with
// the per-chunk partial results kept in a fixed array that is part of the library image:
//
//   * the array holds NFK_ATTN_DECODE_STATIC_SCRATCH_FLOATS floats (8 MiB); every GPU on which the
//     library is loaded carries it from load until the process exits;
//   * a call is rejected with NF_ERR_BAD_ARG (nothing launched) when
//       req_count * q_heads * max_chunks * (head_dim + 2)  exceeds that number;
//   * p->workspace is ignored; inputs, outputs and all other fields mean what they mean for
//     nfk_attn_decode, and chunk_pages == 0 (no split) needs no scratch at all;
//   * the function itself allocates nothing (no cudaMalloc / cudaFree, no allocating library call).
//     The first call on each device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current) and caches it; make that first call
//     before starting any stream capture. The look-up is guarded by a mutex, so first calls from
//     several host threads are safe;
//   * a request with more than chunk_pages * max_chunks pages is still computed in full: its last
//     chunk takes all remaining pages;
//   * all calls on a device share the one array. Nothing in it needs to start at zero: every chunk
//     slot that the merge step reads has been written by the same call. But two calls that overlap
//     on the GPU (different streams) would overwrite each other's partials, so keep calls that use
//     the split path on one stream or order them with events.
#pragma once
#include "kernels.h"

#define NFK_ATTN_DECODE_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

int nfk_attn_decode_static(const nfk_attn_params* p, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
