// Allocation-free variant of the paged decode attention.
//
// This entry point has no counterpart in the reference project. It exists for callers that
// are not allowed to allocate device memory at the time they need attention: code running
// inside a memory pool that another component owns and has already carved up completely,
// plug-ins loaded into a host application whose allocator must not be bypassed, and tight
// serving loops that forbid any allocator call after start-up so that memory use stays flat
// and no call can block on the allocator's implicit device synchronisation.
//
// The split-KV decode kernel needs scratch memory for the per-split partial outputs. The
// regular entry point (pxl_attn_decode in pxl_api.h) takes that scratch from the caller; this
// one keeps it in a fixed array inside the library, so the caller passes only inputs and
// outputs.
#pragma once
#include <stdint.h>

#include "pxl_api.h"

#ifdef __cplusplus
extern "C" {
#endif

// Capacity of the built-in scratch array, in floats (16 MiB). Every GPU that loads the
// library holds this much device memory until the process exits.
#define PXL_DECODE_STATIC_SCRATCH_FLOATS (4 * 1024 * 1024)

// Same computation and arguments as pxl_attn_decode, minus the workspace pointer.
//
//  * Needs B * Hq * num_splits * (D + 2) <= PXL_DECODE_STATIC_SCRATCH_FLOATS when
//    num_splits > 1; larger problems are refused with PXL_ERR_TOO_LARGE (nothing is
//    launched). num_splits must be >= 1 (there is no automatic choice here: the caller
//    decides, so that the size check is predictable).
//  * Calls no cudaMalloc / cudaFree and no allocating library routine.
//  * The first call on each device looks up the device address of the scratch array (once
//    per device, with that device current). Make that first call during set-up, before any
//    stream capture is started.
//  * All calls share the one array. Each call overwrites every scratch element it later reads,
//    so stale contents from an earlier call are harmless and nothing has to be cleared; but
//    two calls whose kernels overlap on the GPU (different streams, or different host threads)
//    would race on it. Issue calls on one stream, or serialise them yourself.
//  * Return value 0 means the kernels were enqueued. After a non-zero return nothing was
//    launched and `out` is untouched. When the kernels ran but the device status word
//    (`status`) is non-zero afterwards - a bounded wait inside the kernel gave up - the
//    contents of `out` are undefined for that call: read the status word before using them.
//  * The per-device address cache is an atomic pointer written without a lock. Two host threads that make
//    their first call on the same device at the same moment both look the address up and
//    both store the same value through an atomic, which is harmless; nothing else in the call is shared
//    between threads except the scratch array itself (previous item).
int pxl_attn_decode_static_scratch(const void* q, int64_t q_stride, const void* k_cache,
                                   const void* v_cache, const int* block_tables,
                                   const int* ctx_lens, void* out, const float* sinks, int B,
                                   int Hq, int Hkv, int D, int page_size, int max_blocks,
                                   int64_t num_blocks, float scale, int window, int num_splits,
                                   int* status, pxl_stream_t stream);

#ifdef __cplusplus
}
#endif
