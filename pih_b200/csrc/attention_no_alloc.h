// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project: it exists for programs that embed the
// kernel pack where cudaMalloc is off limits — under a host that owns all device memory and hands out
// none (a game engine, another inference runtime's plugin slot), after a set-up phase whose end freezes
// the process's device allocations, or in a real-time loop where an allocation's latency or failure
// cannot be tolerated.
//
// It is the split-KV paged attention of pih_paged_attention_mma (attention_mma.cu) with one difference:
// the scratch memory that the kernel needs for its per-split partial results and tickets is not passed
// in by the caller but lives inside the library, in a fixed array in device global memory of
// PIH_NO_ALLOC_SCRATCH_BYTES bytes.  Every GPU on which the library is loaded carries that array until
// the process exits, used or not.
//
// Rules for the caller:
//   * Inputs and outputs are still the caller's (device pointers, as for pih_paged_attention_mma).
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress).  Make
//     that first call outside any stream capture, with the device current; later calls on that device
//     do no set-up.
//   * A problem whose scratch need exceeds the array is refused with PIH_NO_ALLOC_TOO_LARGE and a
//     message in `message` (if given); nothing is launched.  The need is
//     pih_attention_scratch_floats(num_requests, dec_tok_cap, heads, kv_heads, head_dim, max_splits) * 4 bytes.
//   * All calls share the one array per device.  The function clears the part that must start at zero
//     on the given stream before it launches, so leftovers of an earlier (even an aborted) call do not
//     matter — but two calls whose kernels can overlap on the GPU (different streams, no ordering between
//     them) would corrupt each other's partial results.  Serialise them.
//   * The function calls no cudaMalloc, cudaFree or any library routine that allocates.
#pragma once

#include <stdint.h>

#define PIH_NO_ALLOC_SCRATCH_BYTES (8u * 1024u * 1024u)
#define PIH_NO_ALLOC_TOO_LARGE (-3)
#define PIH_NO_ALLOC_SETUP_FAILED (-4)

#ifdef __cplusplus
extern "C" {
#endif

// Arguments as pih_paged_attention_mma, without `scratch`; `split` must be > 0 (keys per split, a multiple
// of 64) so that the scratch need is known on the host.  `message` (nullable) receives a zero-terminated
// explanation when the return value is not 0.  Returns 0, a negative PIH_* code, or a cudaError_t (> 0).
// For tests and diagnostics: the device address of the built-in array on the current device, or null
// before the first call of pih_paged_attention_mma_no_alloc on that device.  It allocates nothing.
void* pih_no_alloc_scratch_address(void);

int pih_paged_attention_mma_no_alloc(const void* q, int q_stride, void* out, const void* cache,
                                     const int* block_table, int table_width, const int* cu_q,
                                     const int* q_start, int rows, int num_requests, int tile_max_q,
                                     int dec_tok_cap, int dec_max_ctx, int heads, int kv_heads, int head_dim,
                                     int page_size, int num_pages, float scale, int window, int split,
                                     const void* kv_tensor_map, uint32_t* error, void* stream, char* message,
                                     int message_capacity);

#ifdef __cplusplus
}
#endif
