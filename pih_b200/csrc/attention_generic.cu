// Causal grouped-query attention over the paged cache on CUDA cores, 32-bit
// arithmetic, any head size, any number of heads and groups, any page size,
// optional sliding window.  It is the attention of the true 32-bit path and
// the plain twin of the tensor-core kernels.
//
// One warp per (query row, query head).  The row at absolute position p
// reads keys first..p with first = max(0, p - window + 1) (0 without a
// window), in blocks of 32 that start at `first`: the order of every
// reduction depends on p and the window alone, never on how the prompt was
// cut into steps, on the other rows of the batch or on which pages hold the
// keys.  Online softmax as the reference's kernel does it
// (kernels/cuda/qwen_bf16_primitives.cu:660-733): score = (q . k) * scale with
// the scale after the dot product, running maximum, running sum,
// accumulator rescaled when the maximum moves, one rounding of acc / sum.
//
// q is read from the fused projection buffer [rows, row_stride] (head h at
// column h * head_dim); cache layout [page][2][kv_head][page_size][head_dim].
#include "common.cuh"

namespace pih {

constexpr int kMaxDimPerLane = 8;   // head_dim <= 256

template <typename T>
__global__ void paged_attention_generic_kernel(
    const T* __restrict__ q, int q_stride, T* __restrict__ out, const T* __restrict__ cache,
    const int* __restrict__ block_table, int table_width, const int* __restrict__ request_of_row,
    const int* __restrict__ positions, int rows, int heads, int kv_heads, int head_dim, int page_size,
    int num_pages, float scale, int window, uint32_t* error) {
  wait_for_prior_kernels();
  launch_dependents();                                   // (the next kernel's blocks may become resident and wait)
  extern __shared__ float smem[];
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = static_cast<long long>(blockIdx.x) * warps_per_block + warp;
  if (item >= static_cast<long long>(rows) * heads) return;
  const int t = static_cast<int>(item / heads);
  const int h = static_cast<int>(item % heads);
  const int g = h / (heads / kv_heads);
  const int r = request_of_row[t];
  if (r < 0) return;                                   // a row of padding
  const int p = positions[t];
  const int first = window > 0 ? max(0, p - window + 1) : 0;
  const int* table = block_table + static_cast<size_t>(r) * table_width;

  float* qs = smem + warp * head_dim;
  const T* qrow = q + static_cast<size_t>(t) * q_stride + static_cast<size_t>(h) * head_dim;
  for (int c = lane; c < head_dim; c += 32) qs[c] = to_float<T>(qrow[c]);
  __syncwarp();

  float acc[kMaxDimPerLane];
#pragma unroll
  for (int i = 0; i < kMaxDimPerLane; ++i) acc[i] = 0.0f;
  float m = -INFINITY, l = 0.0f;
  const size_t head_elems = static_cast<size_t>(page_size) * head_dim;

  for (int base = first; base <= p; base += 32) {
    const int j = base + lane;
    const bool valid = j <= p;
    float s = -INFINITY;
    const T* krow = nullptr;
    if (valid) {
      const int page = table[j / page_size];
      if (page < 0 || page >= num_pages) {
        publish_error(error, kRowWithoutPage);
      } else {
        krow = cache + ((static_cast<size_t>(page) * 2 + 0) * kv_heads + g) * head_elems +
               static_cast<size_t>(j % page_size) * head_dim;
        float dot = 0.0f;
        for (int c = 0; c < head_dim; ++c) dot = fmaf(qs[c], to_float<T>(krow[c]), dot);
        s = dot * scale;
      }
    }
    const float block_max = warp_max(s);
    const float m_new = fmaxf(m, block_max);
    const float alpha = (m == -INFINITY) ? 0.0f : expf(m - m_new);
    const float e = (s == -INFINITY) ? 0.0f : expf(s - m_new);
    l = l * alpha + warp_sum(e);
#pragma unroll
    for (int i = 0; i < kMaxDimPerLane; ++i) acc[i] *= alpha;
    const int count = min(32, p - base + 1);
    for (int jj = 0; jj < count; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, e, jj);
      const int kj = base + jj;
      const int page = table[kj / page_size];
      if (page < 0 || page >= num_pages) continue;     // reported above by the lane that owns kj
      const T* vrow = cache + ((static_cast<size_t>(page) * 2 + 1) * kv_heads + g) * head_elems +
                      static_cast<size_t>(kj % page_size) * head_dim;
#pragma unroll
      for (int i = 0; i < kMaxDimPerLane; ++i) {
        const int c = lane + 32 * i;
        if (c < head_dim) acc[i] = fmaf(pj, to_float<T>(vrow[c]), acc[i]);
      }
    }
    m = m_new;
  }
  if (!(l > 0.0f) || !isfinite(l)) {
    if (lane == 0) publish_error(error, kAttentionDenominator);
    l = 1.0f;
  }
  T* orow = out + (static_cast<size_t>(t) * heads + h) * head_dim;
#pragma unroll
  for (int i = 0; i < kMaxDimPerLane; ++i) {
    const int c = lane + 32 * i;
    if (c < head_dim) orow[c] = from_float<T>(acc[i] / l);
  }
}

}  // namespace pih

using namespace pih;

extern "C" int pih_paged_attention_generic(int dtype, const void* q, int q_stride, void* out,
                                           const void* cache, const int* block_table, int table_width,
                                           const int* request_of_row, const int* positions, int rows,
                                           int heads, int kv_heads, int head_dim, int page_size,
                                           int num_pages, float scale, int window, uint32_t* error,
                                           void* stream) {
  if (rows <= 0) return 0;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || head_dim <= 0 || page_size <= 0 ||
      table_width <= 0 || window < 0)
    return PIH_ERR_BAD_ARGUMENT;
  if (head_dim > 32 * kMaxDimPerLane) return PIH_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int warps = 4;
  const long long items = static_cast<long long>(rows) * heads;
  const unsigned blocks = static_cast<unsigned>((items + warps - 1) / warps);
  const size_t smem = static_cast<size_t>(warps) * head_dim * sizeof(float);
  if (dtype == PIH_F32)
    launch_kernel(paged_attention_generic_kernel<float>, dim3(blocks), dim3(warps * 32), smem, s, 
        static_cast<const float*>(q), q_stride, static_cast<float*>(out),
        static_cast<const float*>(cache), block_table, table_width, request_of_row, positions, rows,
        heads, kv_heads, head_dim, page_size, num_pages, scale, window, error);
  else if (dtype == PIH_BF16)
    launch_kernel(paged_attention_generic_kernel<__nv_bfloat16>, dim3(blocks), dim3(warps * 32), smem, s, 
        static_cast<const __nv_bfloat16*>(q), q_stride, static_cast<__nv_bfloat16*>(out),
        static_cast<const __nv_bfloat16*>(cache), block_table, table_width, request_of_row, positions,
        rows, heads, kv_heads, head_dim, page_size, num_pages, scale, window, error);
  else
    return PIH_ERR_BAD_ARGUMENT;
  PIH_LAUNCH_CHECK();
  return 0;
}
