// See attention_no_alloc.h: split-KV decode attention whose scratch lives in the library.
#include "attention_no_alloc.h"

#include <cuda_runtime.h>
#include <stdio.h>

// the existing entry point and its sizing helpers (attention_mma.cu)
extern "C" long long pih_attention_ticket_words(int num_requests, int kv_heads);
extern "C" long long pih_attention_scratch_floats(int num_requests, int dec_tok_cap, int heads, int kv_heads,
                                                  int head_dim, int max_splits);
extern "C" int pih_paged_attention_mma(const void* q, int q_stride, void* out, const void* cache,
                                       const int* block_table, int table_width, const int* cu_q,
                                       const int* q_start, int rows, int num_requests, int tile_max_q,
                                       int dec_tok_cap, int dec_max_ctx, int heads, int kv_heads, int head_dim,
                                       int page_size, int num_pages, float scale, int window, int split,
                                       int max_splits, const int* max_ctx_ptr, float* scratch,
                                       const void* kv_tensor_map, uint32_t* error, void* stream);

namespace {

// The scratch itself.  In host code this name is only a handle for cudaGetSymbolAddress — it is NOT a
// device address and must never be handed to a kernel as one.
static __device__ __align__(256) float g_attention_scratch[PIH_NO_ALLOC_SCRATCH_BYTES / sizeof(float)];

constexpr int kMaxDevices = 64;
float* g_scratch_address[kMaxDevices] = {};     // per device, filled by the first call on that device

void explain(char* message, int capacity, const char* text) {
  if (message != nullptr && capacity > 0) snprintf(message, static_cast<size_t>(capacity), "%s", text);
}

}  // namespace

extern "C" void* pih_no_alloc_scratch_address(void) {
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return nullptr;
  return g_scratch_address[device];
}

extern "C" int pih_paged_attention_mma_no_alloc(const void* q, int q_stride, void* out, const void* cache,
                                                const int* block_table, int table_width, const int* cu_q,
                                                const int* q_start, int rows, int num_requests, int tile_max_q,
                                                int dec_tok_cap, int dec_max_ctx, int heads, int kv_heads,
                                                int head_dim, int page_size, int num_pages, float scale,
                                                int window, int split, const void* kv_tensor_map, uint32_t* error,
                                                void* stream, char* message, int message_capacity) {
  explain(message, message_capacity, "");
  if (split <= 0 || split % 64 || num_requests <= 0 || heads <= 0 || kv_heads <= 0 || head_dim <= 0 ||
      dec_tok_cap < 0 || dec_max_ctx < 0) {
    explain(message, message_capacity, "bad argument: split must be a positive multiple of 64 and all sizes positive");
    return -1;
  }
  // how much scratch this problem needs, against what the library holds
  const int max_splits = dec_tok_cap > 0 ? (dec_max_ctx + split - 1) / split : 0;
  const long long need_bytes =
      pih_attention_scratch_floats(num_requests, dec_tok_cap, heads, kv_heads, head_dim, max_splits) * 4;
  if (need_bytes > static_cast<long long>(PIH_NO_ALLOC_SCRATCH_BYTES)) {
    if (message != nullptr && message_capacity > 0)
      snprintf(message, static_cast<size_t>(message_capacity),
               "this attention problem needs %lld bytes of scratch, the built-in array holds %u: use fewer requests "
               "or a larger split, or call pih_paged_attention_mma with scratch of your own",
               need_bytes, PIH_NO_ALLOC_SCRATCH_BYTES);
    return PIH_NO_ALLOC_TOO_LARGE;
  }
  // set-up, once per device: the device address of the array
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess || device < 0 || device >= kMaxDevices) {
    explain(message, message_capacity, "cudaGetDevice failed or the device index is out of range");
    return PIH_NO_ALLOC_SETUP_FAILED;
  }
  if (g_scratch_address[device] == nullptr) {
    float* address = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_attention_scratch);
    if (e != cudaSuccess || address == nullptr) {
      if (message != nullptr && message_capacity > 0)
        snprintf(message, static_cast<size_t>(message_capacity), "cudaGetSymbolAddress failed: %s",
                 cudaGetErrorString(e));
      return PIH_NO_ALLOC_SETUP_FAILED;
    }
    g_scratch_address[device] = address;
  }
  float* scratch = g_scratch_address[device];
  // the tickets at the front of the scratch must be zero when the kernel starts; whatever the last call left
  // there (it leaves zeros unless it was cut short) is cleared on the caller's stream
  const long long ticket_bytes = pih_attention_ticket_words(num_requests, kv_heads) * 4;
  e = cudaMemsetAsync(scratch, 0, static_cast<size_t>(ticket_bytes), static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    explain(message, message_capacity, "clearing the tickets failed");
    return static_cast<int>(e);
  }
  const int rc = pih_paged_attention_mma(q, q_stride, out, cache, block_table, table_width, cu_q, q_start, rows,
                                         num_requests, tile_max_q, dec_tok_cap, dec_max_ctx, heads, kv_heads,
                                         head_dim, page_size, num_pages, scale, window, split, 0, nullptr, scratch,
                                         kv_tensor_map, error, stream);
  if (rc != 0) explain(message, message_capacity, "the attention launch was refused or failed; see the return code");
  return rc;
}
