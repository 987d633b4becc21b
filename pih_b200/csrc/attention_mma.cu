// Causal grouped-query attention over the paged cache on tensor cores (bf16
// inputs, fp32 scores, softmax and accumulation), for prompt portions and for
// decode tokens of a mixed batch.
//
// The reference's kernel gives each (query row, head) to ONE THREAD that walks
// all keys (kernels/cuda/qwen_bf16_primitives.cu:620-734, launched with one
// thread per block).  The formula is kept — score = (q . k) * scale, causal
// mask by position, online softmax in 32-bit, one rounding of acc / sum — and
// the execution is new:
//
// * Rows are packed per kv head: packed row i of a request is (token i / G,
//   query head g * G + i % G) with G = heads / kv_heads, so that all query
//   heads that share a kv head share its K and V tiles, for any G.
// * A tile of 16 packed rows per warp runs flash-attention style over key
//   tiles of 64 that are gathered page by page with cp.async into padded
//   shared memory (row stride head_dim + 8 elements keeps ldmatrix free of
//   bank conflicts for every head_dim that is a multiple of 16), two stages.
// * "Tile" kernel (4 warps, 64 packed rows, K/V tiles shared by the warps):
//   requests that bring more than 16 packed rows.
// * "Split" kernel (1 warp, 16 packed rows): requests that bring at most 16
//   packed rows (decode).  The keys are cut at fixed absolute positions
//   (multiples of `split`), one CTA per (split, kv head, request), each writing
//   an unnormalised partial (acc, max, sum) to scratch memory; a combine
//   kernel merges the partials of a row in ascending order.  The cut does not
//   depend on the batch.
//
// mma.sync.m16n8k16 is used rather than tcgen05: the M dimension of a decode
// tile is 2..16 rows, far below the 128-row tcgen05 tile, and the kernel is
// bound by the bandwidth of the cache reads, not by the tensor pipe.
#include "common.cuh"

namespace pih {

constexpr int BN = 64;                 // keys per tile
constexpr float kLog2e = 1.4426950408889634f;

struct AttnParams {
  const __nv_bfloat16* q;
  int q_stride;                        // elements between rows of q
  __nv_bfloat16* out;                  // [rows, heads * D]
  const __nv_bfloat16* cache;          // [page][2][kv_head][page_size][D]
  const int* block_table;              // [R, table_width]
  int table_width;
  const int* cu_q;                     // [R + 1]
  const int* q_start;                  // [R] position of a request's first row
  int heads, kv_heads, page_size, num_pages;
  float scale;
  int window;                          // 0: none
  int split;                           // keys per split (split kernel)
  int max_splits;
  int dec_tok_cap;                     // most rows of one decode-like request
  float* part_o;                       // [R, dec_tok_cap, heads, max_splits, D]
  float* part_ml;                      // [R, dec_tok_cap, heads, max_splits, 2]
  uint32_t* error;
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, int src_bytes) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Gather one tile of BN keys (K and V of kv head g) starting at key j0 into shared memory.
// Keys outside [kmin, kmax] are zero-filled and never read from the cache.
template <int D, int THREADS>
__device__ __forceinline__ void load_kv_tile(const AttnParams& p, const int* table, int g, int j0, int kmin,
                                             int kmax, __nv_bfloat16* Ks, __nv_bfloat16* Vs) {
  constexpr int LD = D + 8;
  constexpr int CHUNKS = D / 8;                      // 16-byte chunks per row
  const size_t head_elems = static_cast<size_t>(p.page_size) * D;
  for (int c = threadIdx.x; c < BN * CHUNKS; c += THREADS) {
    const int row = c / CHUNKS, ch = c % CHUNKS;
    const int j = j0 + row;
    const __nv_bfloat16* ksrc = p.cache;
    const __nv_bfloat16* vsrc = p.cache;
    int bytes = 0;
    if (j >= kmin && j <= kmax) {
      const int page = table[j / p.page_size];
      if (page < 0 || page >= p.num_pages) {
        publish_error(p.error, kRowWithoutPage);
      } else {
        const size_t base = (static_cast<size_t>(page) * 2 * p.kv_heads + g) * head_elems +
                            static_cast<size_t>(j % p.page_size) * D + ch * 8;
        ksrc = p.cache + base;
        vsrc = p.cache + base + static_cast<size_t>(p.kv_heads) * head_elems;
        bytes = 16;
      }
    }
    cp_async16(Ks + row * LD + ch * 8, ksrc, bytes);
    cp_async16(Vs + row * LD + ch * 8, vsrc, bytes);
  }
}

// One warp: 16 packed rows against one tile of BN keys.
template <int D>
__device__ __forceinline__ void tile_step(const __nv_bfloat16* Qs /* this warp's 16 rows */,
                                          const __nv_bfloat16* Ks, const __nv_bfloat16* Vs, int j0,
                                          const int (&row_pos)[2], const int (&row_first)[2], float scale_log2,
                                          float (&m)[2], float (&l)[2], float (&o)[D / 8][4]) {
  constexpr int LD = D + 8;
  const int lane = threadIdx.x & 31;
  float s[BN / 8][4];
#pragma unroll
  for (int n = 0; n < BN / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
  // S = Q K^T
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    uint32_t a[4];
    ldmatrix_x4(a, Qs + ((lane & 7) + ((lane >> 3) & 1) * 8) * LD + kk * 16 + (lane >> 4) * 8);
#pragma unroll
    for (int nt = 0; nt < BN / 16; ++nt) {
      uint32_t b[4];
      ldmatrix_x4(b, Ks + (nt * 16 + (lane & 7) + (lane >> 4) * 8) * LD + kk * 16 + ((lane >> 3) & 1) * 8);
      mma_bf16(s[2 * nt], a, b[0], b[1]);
      mma_bf16(s[2 * nt + 1], a, b[2], b[3]);
    }
  }
  // scale, mask, online softmax (base 2)
  float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = e >> 1;
      const int j = j0 + n * 8 + (lane & 3) * 2 + (e & 1);
      const bool visible = j <= row_pos[r] && j >= row_first[r];
      const float v = visible ? s[n][e] * scale_log2 : -INFINITY;
      s[n][e] = v;
      tile_max[r] = fmaxf(tile_max[r], v);
    }
  }
  float alpha[2], m_use[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
    tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
    const float m_new = fmaxf(m[r], tile_max[r]);
    m_use[r] = (m_new == -INFINITY) ? 0.0f : m_new;
    alpha[r] = (m[r] == -INFINITY) ? 0.0f : exp2f(m[r] - m_use[r]);
    m[r] = m_new;
  }
  float tile_sum[2] = {0.0f, 0.0f};
#pragma unroll
  for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = e >> 1;
      const float pv = exp2f(s[n][e] - m_use[r]);        // exp2(-inf) = 0 for masked keys
      s[n][e] = pv;
      tile_sum[r] += pv;
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) l[r] = l[r] * alpha[r] + tile_sum[r];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) {
    o[n][0] *= alpha[0];
    o[n][1] *= alpha[0];
    o[n][2] *= alpha[1];
    o[n][3] *= alpha[1];
  }
  // O += P V
#pragma unroll
  for (int kk = 0; kk < BN / 16; ++kk) {
    uint32_t a[4];
    a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
    for (int nt = 0; nt < D / 16; ++nt) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, Vs + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + nt * 16 + (lane >> 4) * 8);
      mma_bf16(o[2 * nt], a, b[0], b[1]);
      mma_bf16(o[2 * nt + 1], a, b[2], b[3]);
    }
  }
}

// NWARPS = 4: tile kernel, grid (q tiles, kv_heads, R).  NWARPS = 1: split kernel, grid (splits, kv_heads, R).
template <int D, int NWARPS, bool SPLIT>
__global__ void __launch_bounds__(NWARPS * 32)
attn_mma_kernel(const AttnParams p) {
  constexpr int LD = D + 8;
  constexpr int BM = NWARPS * 16;
  constexpr int THREADS = NWARPS * 32;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* Ks0 = Qs + BM * LD;
  __nv_bfloat16* Vs0 = Ks0 + 2 * BN * LD;

  const int r = blockIdx.z, g = blockIdx.y;
  const int G = p.heads / p.kv_heads;
  const int row0 = p.cu_q[r];
  const int n_tok = p.cu_q[r + 1] - row0;
  const int packed = n_tok * G;
  const bool decode_like = packed <= 16;
  if (SPLIT != decode_like) return;
  const int tile_row0 = SPLIT ? 0 : blockIdx.x * BM;
  if (tile_row0 >= packed) return;
  const int start = p.q_start[r];
  // key range that the rows of this tile can see
  const int tok_lo = tile_row0 / G;
  const int tok_hi = min(packed - 1, tile_row0 + BM - 1) / G;
  int kmin = p.window > 0 ? max(0, start + tok_lo - p.window + 1) : 0;
  int kmax = start + tok_hi;
  if (SPLIT) {
    kmin = max(kmin, static_cast<int>(blockIdx.x) * p.split);
    kmax = min(kmax, (static_cast<int>(blockIdx.x) + 1) * p.split - 1);
    if (kmin > kmax) return;
  }
  const int* table = p.block_table + static_cast<size_t>(r) * p.table_width;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // Q tile
  for (int c = threadIdx.x; c < BM * (D / 8); c += THREADS) {
    const int row = c / (D / 8), ch = c % (D / 8);
    const int i = tile_row0 + row;
    const bool valid = i < packed;
    const __nv_bfloat16* src = p.q;
    if (valid)
      src = p.q + static_cast<size_t>(row0 + i / G) * p.q_stride + static_cast<size_t>(g * G + i % G) * D + ch * 8;
    cp_async16(Qs + row * LD + ch * 8, src, valid ? 16 : 0);
  }
  const int t_first = kmin / BN, t_last = kmax / BN;
  load_kv_tile<D, THREADS>(p, table, g, t_first * BN, kmin, kmax, Ks0, Vs0);
  cp_async_commit();

  // the two rows this thread owns in the accumulator layout
  int row_pos[2], row_first[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int i = tile_row0 + warp * 16 + (lane >> 2) + h * 8;
    if (i < packed) {
      row_pos[h] = start + i / G;
      row_first[h] = p.window > 0 ? max(0, row_pos[h] - p.window + 1) : 0;
    } else {
      row_pos[h] = -1;                 // sees nothing
      row_first[h] = 0;
    }
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
  const float scale_log2 = p.scale * kLog2e;

  for (int t = t_first; t <= t_last; ++t) {
    const int buf = (t - t_first) & 1;
    if (t < t_last) {
      load_kv_tile<D, THREADS>(p, table, g, (t + 1) * BN, kmin, kmax, Ks0 + (buf ^ 1) * BN * LD,
                               Vs0 + (buf ^ 1) * BN * LD);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    tile_step<D>(Qs + warp * 16 * LD, Ks0 + buf * BN * LD, Vs0 + buf * BN * LD, t * BN, row_pos, row_first,
                 scale_log2, m, l, o);
    __syncthreads();
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int i = tile_row0 + warp * 16 + (lane >> 2) + h * 8;
    if (i >= packed) continue;
    const int grow = row0 + i / G, head = g * G + i % G;
    if (SPLIT) {
      const size_t slot =
          ((static_cast<size_t>(r) * p.dec_tok_cap + i / G) * p.heads + head) * p.max_splits + blockIdx.x;
      float* po = p.part_o + slot * D;
#pragma unroll
      for (int n = 0; n < D / 8; ++n) {
        const int d = n * 8 + (lane & 3) * 2;
        *reinterpret_cast<float2*>(po + d) = make_float2(o[n][2 * h], o[n][2 * h + 1]);
      }
      if ((lane & 3) == 0) {
        p.part_ml[slot * 2] = m[h];
        p.part_ml[slot * 2 + 1] = l[h];
      }
    } else {
      if (!(l[h] > 0.0f) || !isfinite(l[h])) {
        publish_error(p.error, kAttentionDenominator);
        continue;
      }
      const float inv = 1.0f / l[h];
      __nv_bfloat16* orow = p.out + (static_cast<size_t>(grow) * p.heads + head) * D;
#pragma unroll
      for (int n = 0; n < D / 8; ++n) {
        const int d = n * 8 + (lane & 3) * 2;
        *reinterpret_cast<uint32_t*>(orow + d) = pack_bf16(o[n][2 * h] * inv, o[n][2 * h + 1] * inv);
      }
    }
  }
}

// Merge the partials of each decode-like row in ascending split order.  One warp per (row, head).
__global__ void attn_combine_kernel(const AttnParams p, int rows, int head_dim, const int* request_of_row,
                                    const int* positions) {
  const int warps = blockDim.x >> 5;
  const long long item = static_cast<long long>(blockIdx.x) * warps + (threadIdx.x >> 5);
  if (item >= static_cast<long long>(rows) * p.heads) return;
  const int lane = threadIdx.x & 31;
  const int t = static_cast<int>(item / p.heads), h = static_cast<int>(item % p.heads);
  const int r = request_of_row[t];
  const int G = p.heads / p.kv_heads;
  if ((p.cu_q[r + 1] - p.cu_q[r]) * G > 16) return;              // not a decode-like request
  const int pos = positions[t];
  const int first = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  const int s_lo = first / p.split, s_hi = pos / p.split;
  const size_t base =
      ((static_cast<size_t>(r) * p.dec_tok_cap + (t - p.cu_q[r])) * p.heads + h) * p.max_splits;
  float m = -INFINITY;
  for (int s = s_lo; s <= s_hi; ++s) m = fmaxf(m, p.part_ml[(base + s) * 2]);
  float l = 0.0f;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
  for (int s = s_lo; s <= s_hi; ++s) {
    const float ms = p.part_ml[(base + s) * 2];
    if (ms == -INFINITY) continue;
    const float w = exp2f(ms - m);
    l += p.part_ml[(base + s) * 2 + 1] * w;
    const float* po = p.part_o + (base + s) * head_dim;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int d = lane + 32 * i;
      if (d < head_dim) acc[i] += po[d] * w;
    }
  }
  if (!(l > 0.0f) || !isfinite(l)) {
    if (lane == 0) publish_error(p.error, kAttentionDenominator);
    return;
  }
  __nv_bfloat16* orow = p.out + (static_cast<size_t>(t) * p.heads + h) * head_dim;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int d = lane + 32 * i;
    if (d < head_dim) orow[d] = __float2bfloat16_rn(acc[i] / l);
  }
}

template <int D, int NWARPS, bool SPLIT>
static int launch_attn(const AttnParams& p, dim3 grid, cudaStream_t s) {
  constexpr int LD = D + 8;
  constexpr int BM = NWARPS * 16;
  const int smem = (BM * LD + 4 * BN * LD) * static_cast<int>(sizeof(__nv_bfloat16));
  static bool configured = false;            // per template instance
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_mma_kernel<D, NWARPS, SPLIT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  attn_mma_kernel<D, NWARPS, SPLIT><<<grid, NWARPS * 32, smem, s>>>(p);
  PIH_LAUNCH_CHECK();
  return 0;
}

template <int D>
static int launch_both(const AttnParams& p, int R, int tile_max_q, int rows, const int* request_of_row,
                       const int* positions, cudaStream_t s) {
  const int G = p.heads / p.kv_heads;
  if (tile_max_q > 0) {
    dim3 grid((tile_max_q * G + 63) / 64, p.kv_heads, R);
    const int rc = launch_attn<D, 4, false>(p, grid, s);
    if (rc) return rc;
  }
  if (p.dec_tok_cap > 0) {
    dim3 grid(p.max_splits, p.kv_heads, R);
    int rc = launch_attn<D, 1, true>(p, grid, s);
    if (rc) return rc;
    const int warps = 4;
    const long long items = static_cast<long long>(rows) * p.heads;
    attn_combine_kernel<<<static_cast<unsigned>((items + warps - 1) / warps), warps * 32, 0, s>>>(
        p, rows, D, request_of_row, positions);
    PIH_LAUNCH_CHECK();
  }
  return 0;
}

}  // namespace pih

using namespace pih;

// Floats of scratch that the split kernel needs.
extern "C" long long pih_attention_scratch_floats(int num_requests, int dec_tok_cap, int heads, int head_dim,
                                                  int max_splits) {
  return static_cast<long long>(num_requests) * dec_tok_cap * heads * max_splits * (head_dim + 2);
}

// A request is "decode-like" when it brings at most 16 packed rows (rows * heads / kv_heads <= 16).
//   tile_max_q   the most rows of a request that is NOT decode-like (0: there is none)
//   dec_tok_cap  the most rows of a decode-like request (0: there is none)
//   dec_max_ctx  the longest context (after the step) of a decode-like request
// scratch holds pih_attention_scratch_floats(num_requests, dec_tok_cap, heads, head_dim,
// ceil(dec_max_ctx / split)) floats.  Returns PIH_ERR_UNSUPPORTED for a head_dim that has no
// tensor-core instance (the caller then uses the generic kernel).
extern "C" int pih_paged_attention_mma(const void* q, int q_stride, void* out, const void* cache,
                                       const int* block_table, int table_width, const int* cu_q,
                                       const int* q_start, const int* request_of_row, const int* positions,
                                       int rows, int num_requests, int tile_max_q, int dec_tok_cap,
                                       int dec_max_ctx, int heads, int kv_heads, int head_dim, int page_size,
                                       int num_pages, float scale, int window, int split, float* scratch,
                                       uint32_t* error, void* stream) {
  if (rows <= 0) return 0;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || page_size <= 0 || table_width <= 0 || window < 0 ||
      split <= 0 || split % BN || num_requests <= 0 || num_requests > 65535 || kv_heads > 65535 ||
      q_stride % 8 || tile_max_q < 0 || dec_tok_cap < 0 || (dec_tok_cap > 0 && (dec_max_ctx <= 0 || !scratch)))
    return PIH_ERR_BAD_ARGUMENT;
  AttnParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.q_stride = q_stride;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.cache = static_cast<const __nv_bfloat16*>(cache);
  p.block_table = block_table;
  p.table_width = table_width;
  p.cu_q = cu_q;
  p.q_start = q_start;
  p.heads = heads;
  p.kv_heads = kv_heads;
  p.page_size = page_size;
  p.num_pages = num_pages;
  p.scale = scale;
  p.window = window;
  p.split = split;
  p.max_splits = dec_tok_cap > 0 ? (dec_max_ctx + split - 1) / split : 0;
  p.dec_tok_cap = dec_tok_cap;
  p.part_o = scratch;
  p.part_ml = scratch + static_cast<size_t>(num_requests) * dec_tok_cap * heads * p.max_splits * head_dim;
  p.error = error;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (head_dim) {
    case 16: return launch_both<16>(p, num_requests, tile_max_q, rows, request_of_row, positions, s);
    case 32: return launch_both<32>(p, num_requests, tile_max_q, rows, request_of_row, positions, s);
    case 64: return launch_both<64>(p, num_requests, tile_max_q, rows, request_of_row, positions, s);
    case 80: return launch_both<80>(p, num_requests, tile_max_q, rows, request_of_row, positions, s);
    case 96: return launch_both<96>(p, num_requests, tile_max_q, rows, request_of_row, positions, s);
    case 128: return launch_both<128>(p, num_requests, tile_max_q, rows, request_of_row, positions, s);
    case 256: return launch_both<256>(p, num_requests, tile_max_q, rows, request_of_row, positions, s);
    default: return PIH_ERR_UNSUPPORTED;
  }
}
