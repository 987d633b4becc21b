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
// * "Split" kernel (4 warps, 16 packed rows): requests that bring at most 16
//   packed rows (decode).  The keys are cut at fixed absolute positions
//   (multiples of `split`), one CTA per (split, kv head, request).  All tiles
//   of a split are requested at once (cp.async), the four warps take a
//   quarter of each tile's keys, merge through shared memory and write an
//   unnormalised partial (acc, max, sum) to scratch memory.  The CTA that
//   finishes last for its (request, kv head) — found with one atomic ticket —
//   merges the partials in ascending split order and writes the output, so
//   no second launch is needed and the order of the merge is fixed.  The cut
//   does not depend on the batch.
//
// mma.sync.m16n8k16 is used rather than tcgen05: the M dimension of a decode
// tile is 2..16 rows, far below the 128-row tcgen05 tile, and the kernel is
// bound by the bandwidth of the cache reads, not by the tensor pipe.
#include <string.h>

#include "ptx.cuh"
#include "qk_math.cuh"

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
  int split;                           // keys per split (split kernel); 0: derived on the device, see split_of
  const int* max_ctx_ptr;              // device word: the longest context of this step (used when split == 0)
  int max_splits;                      // grid.x of the split kernel = splits per request at most
  int dec_tok_cap;                     // most rows of one decode-like request
  float* part_o;                       // [R, dec_tok_cap, heads, max_splits, D]
  float* part_ml;                      // [R, dec_tok_cap, heads, max_splits, 2]
  int* tickets;                        // [R, kv_heads], zero between launches
  int page_shift;                      // log2(page_size) or -1
  uint32_t* error;
  // when the split kernel does the q/k norm, the rotation and the cache append itself (FUSE): q points at the raw
  // rows [q | k | v] of the q/k/v product
  const void* q_norm_w;                // [D] or nullptr
  const void* k_norm_w;
  int norm_w_f32;                      // the norm weights are float (else bf16)
  float norm_eps;
  const float* rope;                   // [max_pos, D / 2, 2] (cos, sin) or nullptr
  int max_pos;
  int write_kv;                        // append the new tokens' k and v to the cache (and use them)
  __nv_bfloat16* cache_w;              // the cache, writable
  int fused;                           // host: launch the FUSE variant
  int push_merge;                      // host: the cluster's blocks send their partials to the blocks that finish them
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

// Keys per split.  Either fixed by the host, or the context of the step cut into max_splits equal parts
// (rounded up to whole tiles): then the grid depends on the batch size alone and the cut follows the
// context as it grows, which a captured CUDA graph needs.  At least two tiles per split: with one tile a
// block's fixed costs (set-up, the merge of the splits) outweigh what the extra blocks bring (one request of
// 2048 keys, 8 kv heads: 15.3 us with 64-key splits, 11.2 us with 128, 11.8 us with 256).
__device__ __forceinline__ int split_of(const AttnParams& p) {
  if (p.split > 0) return p.split;
  const int ctx = max(*p.max_ctx_ptr, 1);
  const int per = (ctx + p.max_splits - 1) / p.max_splits;
  return max(2 * BN, (per + BN - 1) / BN * BN);
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
      const int pidx = p.page_shift >= 0 ? (j >> p.page_shift) : (j / p.page_size);
      const int poff = j - pidx * p.page_size;
      const int page = table[pidx];
      if (page < 0 || page >= p.num_pages) {
        publish_error(p.error, kRowWithoutPage);
      } else {
        const size_t base = (static_cast<size_t>(page) * 2 * p.kv_heads + g) * head_elems +
                            static_cast<size_t>(poff) * D + ch * 8;
        ksrc = p.cache + base;
        vsrc = p.cache + base + static_cast<size_t>(p.kv_heads) * head_elems;
        bytes = 16;
      }
    }
    cp_async16(Ks + row * LD + ch * 8, ksrc, bytes);
    cp_async16(Vs + row * LD + ch * 8, vsrc, bytes);
  }
}

// Element (row, col) of a K or V tile in shared memory, col a multiple of 8.
//   SWZ = false: rows of D + 8 elements (what the cp.async gather writes);
//   SWZ = true:  what TMA writes with the 128-byte swizzle: the tile is D / 64 panels of BN rows x 128
//                bytes, and within a row the 16-byte chunk c sits at c ^ (row & 7).
template <int D, bool SWZ>
__device__ __forceinline__ const __nv_bfloat16* kv_at(const __nv_bfloat16* base, int row, int col) {
  if (SWZ) {
    const char* b = reinterpret_cast<const char*>(base) + (col >> 6) * (BN * 128) + row * 128 +
                    ((((col & 63) >> 3) ^ (row & 7)) << 4);
    return reinterpret_cast<const __nv_bfloat16*>(b);
  }
  return base + row * (D + 8) + col;
}

// One warp: 16 packed rows against the NK keys that start at row key_off of the tile Ks / Vs; j0 is
// the position of the first of them.
template <int D, int NK, bool SWZ>
__device__ __forceinline__ void tile_step(const __nv_bfloat16* Qs /* this warp's 16 rows */,
                                          const __nv_bfloat16* Ks, const __nv_bfloat16* Vs, int key_off, int j0,
                                          const int (&row_pos)[2], const int (&row_first)[2], float scale_log2,
                                          float (&m)[2], float (&l)[2], float (&o)[D / 8][4]) {
  constexpr int LD = D + 8;
  const int lane = threadIdx.x & 31;
  float s[NK / 8][4];
#pragma unroll
  for (int n = 0; n < NK / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
  // S = Q K^T
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    uint32_t a[4];
    ldmatrix_x4(a, Qs + ((lane & 7) + ((lane >> 3) & 1) * 8) * LD + kk * 16 + (lane >> 4) * 8);
#pragma unroll
    for (int nt = 0; nt < NK / 16; ++nt) {
      uint32_t b[4];
      ldmatrix_x4(b, kv_at<D, SWZ>(Ks, key_off + nt * 16 + (lane & 7) + (lane >> 4) * 8,
                                   kk * 16 + ((lane >> 3) & 1) * 8));
      mma_bf16(s[2 * nt], a, b[0], b[1]);
      mma_bf16(s[2 * nt + 1], a, b[2], b[3]);
    }
  }
  // scale, mask, online softmax (base 2)
  float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int n = 0; n < NK / 8; ++n) {
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
  for (int n = 0; n < NK / 8; ++n) {
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
  for (int kk = 0; kk < NK / 16; ++kk) {
    uint32_t a[4];
    a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
    for (int nt = 0; nt < D / 16; ++nt) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, kv_at<D, SWZ>(Vs, key_off + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8,
                                         nt * 16 + (lane >> 4) * 8));
      mma_bf16(o[2 * nt], a, b[0], b[1]);
      mma_bf16(o[2 * nt + 1], a, b[2], b[3]);
    }
  }
}

// Tile kernel: 4 warps, 64 packed rows, grid (q tiles, kv_heads, R); requests with more than 16 packed rows.
template <int D>
__global__ void __launch_bounds__(128)
attn_tile_kernel(const AttnParams p) {
  wait_for_prior_kernels();
  launch_dependents();                                   // (the next kernel's blocks may become resident and wait)
  constexpr int LD = D + 8;
  constexpr int BM = 64;
  constexpr int THREADS = 128;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* Ks0 = Qs + BM * LD;
  __nv_bfloat16* Vs0 = Ks0 + 2 * BN * LD;

  const int r = blockIdx.z, g = blockIdx.y;
  const int G = p.heads / p.kv_heads;
  const int row0 = p.cu_q[r];
  const int n_tok = p.cu_q[r + 1] - row0;
  const int packed = n_tok * G;
  if (packed <= 16) return;                          // decode-like: the split kernel's
  const int tile_row0 = blockIdx.x * BM;
  if (tile_row0 >= packed) return;
  const int start = p.q_start[r];
  // key range that the rows of this tile can see
  const int tok_lo = tile_row0 / G;
  const int tok_hi = min(packed - 1, tile_row0 + BM - 1) / G;
  const int kmin = p.window > 0 ? max(0, start + tok_lo - p.window + 1) : 0;
  const int kmax = start + tok_hi;
  const int* table = p.block_table + static_cast<size_t>(r) * p.table_width;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

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
    tile_step<D, BN, false>(Qs + warp * 16 * LD, Ks0 + buf * BN * LD, Vs0 + buf * BN * LD, 0, t * BN, row_pos,
                            row_first, scale_log2, m, l, o);
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

// The end of a split CTA: merge the four consumer warps through shared memory, write the split's
// partial, draw a ticket, and — in the CTA that draws the last ticket of its (request, kv head) —
// merge all splits in ascending order and write the output.  Called by every thread of the CTA
// (threads beyond the first 128 only take part in the barriers).  `scratch` is shared memory that is
// no longer needed, at least (4 * 16 * D + 128) and (16 * splits + 16) floats.
template <int D>
__device__ __forceinline__ void split_finish(const AttnParams& p, int r, int g, int sp, int s_lo, int s_hi,
                                             int packed, int G, int row0, float (&m)[2], float (&l)[2],
                                             float (&o)[D / 8][4], float* scratch, int* s_last) {
  constexpr int THREADS = 128;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
  }
  // merge the four warps through shared memory (the K/V tiles are no longer needed)
  __syncthreads();
  float* Ow = scratch;          // [4][16][D]
  float* Mw = Ow + 4 * 16 * D;                       // [4][16]
  float* Lw = Mw + 4 * 16;                           // [4][16]
#pragma unroll
  for (int h = 0; h < 2 && warp < 4; ++h) {
    const int row = (lane >> 2) + h * 8;
    float* orow = Ow + (warp * 16 + row) * D;
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      const int d = n * 8 + (lane & 3) * 2;
      *reinterpret_cast<float2*>(orow + d) = make_float2(o[n][2 * h], o[n][2 * h + 1]);
    }
    if ((lane & 3) == 0) {
      Mw[warp * 16 + row] = m[h];
      Lw[warp * 16 + row] = l[h];
    }
  }
  __syncthreads();
  const bool single = s_lo == s_hi;                    // the request fits one split: no partials, no ticket
  for (int idx = threadIdx.x; idx < packed * D && threadIdx.x < THREADS; idx += THREADS) {
    const int row = idx / D, d = idx % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, Mw[w * 16 + row]);
    float acc = 0.0f, ll = 0.0f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = Mw[w * 16 + row];
      if (mw == -INFINITY) continue;
      const float f = exp2f(mw - mm);
      acc += Ow[(w * 16 + row) * D + d] * f;
      ll += Lw[w * 16 + row] * f;
    }
    if (single) {
      if (!(ll > 0.0f) || !isfinite(ll)) {
        publish_error(p.error, kAttentionDenominator);
        continue;
      }
      p.out[(static_cast<size_t>(row0 + row / G) * p.heads + g * G + row % G) * D + d] =
          __float2bfloat16_rn(acc / ll);
      continue;
    }
    const size_t slot =
        ((static_cast<size_t>(r) * p.dec_tok_cap + row / G) * p.heads + g * G + row % G) * p.max_splits + sp;
    p.part_o[slot * D + d] = acc;
    if (d == 0) {
      p.part_ml[slot * 2] = mm;
      p.part_ml[slot * 2 + 1] = ll;
    }
  }
  if (single) return;
  // one ticket per CTA; the CTA that draws the last one merges the splits
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int ticket = atomicAdd(&p.tickets[r * p.kv_heads + g], 1);
    *s_last = ticket == (s_hi - s_lo);
  }
  __syncthreads();
  if (!*s_last) return;
  __threadfence();
  // Final merge over the splits, ascending.  Every (row, split)'s maximum and sum come in with one pass of
  // independent loads; the weights exp2(m_s - M) are formed from shared memory; then every output element is
  // a short sum whose loads are issued in batches.  (No load here waits for another: with the sums fetched
  // one by one inside the per-row loop, a merge of 16 splits cost 8 us.)
  const int nsp = s_hi - s_lo + 1;
  float* Fw = scratch;          // [16][nsp] maxima, then weights
  float* Ls = Fw + 16 * nsp;    // [16][nsp] sums
  float* Lsum = Ls + 16 * nsp;  // [16]
  for (int idx = threadIdx.x; idx < packed * nsp && threadIdx.x < THREADS; idx += THREADS) {
    const int row = idx / nsp, s = s_lo + idx % nsp;
    const size_t slot =
        ((static_cast<size_t>(r) * p.dec_tok_cap + row / G) * p.heads + g * G + row % G) * p.max_splits + s;
    const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml + slot * 2));
    Fw[row * nsp + (s - s_lo)] = ml.x;
    Ls[row * nsp + (s - s_lo)] = ml.y;
  }
  __syncthreads();
  if (threadIdx.x < packed) {
    const int row = threadIdx.x;
    float mm = -INFINITY;
    for (int s = 0; s < nsp; ++s) mm = fmaxf(mm, Fw[row * nsp + s]);
    float ll = 0.0f;
    for (int s = 0; s < nsp; ++s) {
      const float ms = Fw[row * nsp + s];
      const float f = ms == -INFINITY ? 0.0f : exp2f(ms - mm);
      Fw[row * nsp + s] = f;
      ll += f == 0.0f ? 0.0f : Ls[row * nsp + s] * f;
    }
    Lsum[row] = ll;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < packed * D && threadIdx.x < THREADS; idx += THREADS) {
    const int row = idx / D, d = idx % D;
    const size_t base =
        ((static_cast<size_t>(r) * p.dec_tok_cap + row / G) * p.heads + g * G + row % G) * p.max_splits + s_lo;
    const float* po = p.part_o + base * D + d;
    const float* fw = Fw + row * nsp;
    float acc = 0.0f;
    int s = 0;
    for (; s + 8 <= nsp; s += 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = fw[s + u] == 0.0f ? 0.0f : __ldcg(po + static_cast<size_t>(s + u) * D);
#pragma unroll
      for (int u = 0; u < 8; ++u) acc += v[u] * fw[s + u];
    }
    for (; s < nsp; ++s) acc += fw[s] == 0.0f ? 0.0f : __ldcg(po + static_cast<size_t>(s) * D) * fw[s];
    const float ll = Lsum[row];
    if (!(ll > 0.0f) || !isfinite(ll)) {
      publish_error(p.error, kAttentionDenominator);
      continue;
    }
    p.out[(static_cast<size_t>(row0 + row / G) * p.heads + g * G + row % G) * D + d] =
        __float2bfloat16_rn(acc / ll);
  }
  if (threadIdx.x == 0) p.tickets[r * p.kv_heads + g] = 0;     // ready for the next launch
}

constexpr int kMaxCluster = 8;           // the portable cluster size

// Thread-block clusters: the rank of this block in its cluster, the cluster-wide barrier (every thread of
// every block of the cluster executes it; a hardware barrier, nothing spins) and a load from the shared
// memory of another block of the cluster, at the address that `local` has in this block's.
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float load_from_cluster_block(const float* local, uint32_t rank) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(local));
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(a), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// The end of a split block whose (request, kv head) is one cluster: every block merges its four consumer
// warps into a partial in its own shared memory; after a cluster barrier every block reads, for its share of
// the output elements, the partials of all blocks through distributed shared memory, merges them in ascending
// order and writes the output; a second barrier keeps every block (and its shared memory) alive until all have read.
// No partial goes through global memory and nothing is counted with atomics: at batch 8 and 2048-token
// contexts the ticket scheme spent 5 us between the last tile and the last store, of a kernel of 18.
// Called by every thread of every block of the cluster, blocks without keys included (they contribute an
// empty partial).  `scratch` is shared memory that is no longer needed, (4 * 16 * D + 128 + 16 * D + 32) floats.
template <int D>
__device__ __forceinline__ void cluster_finish(const AttnParams& p, int g, int nsp, int packed, int G, int row0,
                                               float (&m)[2], float (&l)[2], float (&o)[D / 8][4],
                                               float* scratch) {
  constexpr int THREADS = 128;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
  }
  __syncthreads();                                   // the K/V tiles are no longer needed
  float* Ow = scratch;                               // [4][16][D]
  float* Mw = Ow + 4 * 16 * D;                       // [4][16]
  float* Lw = Mw + 4 * 16;                           // [4][16]
  float* Po = Lw + 4 * 16;                           // [16][D]   this block's partial
  float* Pml = Po + 16 * D;                          // [16][2]
#pragma unroll
  for (int h = 0; h < 2 && warp < 4; ++h) {
    const int row = (lane >> 2) + h * 8;
    if (row >= packed) continue;
    float* orow = Ow + (warp * 16 + row) * D;
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      const int d = n * 8 + (lane & 3) * 2;
      *reinterpret_cast<float2*>(orow + d) = make_float2(o[n][2 * h], o[n][2 * h + 1]);
    }
    if ((lane & 3) == 0) {
      Mw[warp * 16 + row] = m[h];
      Lw[warp * 16 + row] = l[h];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < packed * D && threadIdx.x < THREADS; idx += THREADS) {
    const int row = idx / D, d = idx % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, Mw[w * 16 + row]);
    float acc = 0.0f, ll = 0.0f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = Mw[w * 16 + row];
      if (mw == -INFINITY) continue;
      const float f = exp2f(mw - mm);
      acc += Ow[(w * 16 + row) * D + d] * f;
      ll += Lw[w * 16 + row] * f;
    }
    Po[row * D + d] = acc;
    if (d == 0) {
      Pml[row * 2] = mm;
      Pml[row * 2 + 1] = ll;
    }
  }
  cluster_sync();                                    // every block's partial is in place
  // Every block finishes its share of the output elements: it reads that element's partial, and its row's
  // maximum and sum, from every block of the cluster — loads that do not depend on one another, so the whole
  // merge costs one trip through distributed shared memory — and adds them in ascending block order.
  const int total = packed * D;
  const int share = (total + nsp - 1) / nsp;
  const int first = static_cast<int>(cluster_rank()) * share;
  for (int idx = first + threadIdx.x; idx < min(total, first + share); idx += blockDim.x) {
    const int row = idx / D, d = idx % D;
    float pm[kMaxCluster], pl[kMaxCluster], po[kMaxCluster];
#pragma unroll
    for (int c = 0; c < kMaxCluster; ++c) {
      pm[c] = -INFINITY;
      pl[c] = po[c] = 0.0f;
      if (c < nsp) {
        pm[c] = load_from_cluster_block(Pml + row * 2, c);
        pl[c] = load_from_cluster_block(Pml + row * 2 + 1, c);
        po[c] = load_from_cluster_block(Po + row * D + d, c);
      }
    }
    float mm = -INFINITY;
#pragma unroll
    for (int c = 0; c < kMaxCluster; ++c) mm = fmaxf(mm, pm[c]);
    float acc = 0.0f, ll = 0.0f;
#pragma unroll
    for (int c = 0; c < kMaxCluster; ++c) {
      if (pm[c] == -INFINITY) continue;
      const float f = exp2f(pm[c] - mm);
      acc += po[c] * f;
      ll += pl[c] * f;
    }
    if (!(ll > 0.0f) || !isfinite(ll)) {
      publish_error(p.error, kAttentionDenominator);
      continue;
    }
    p.out[(static_cast<size_t>(row0 + row / G) * p.heads + g * G + row % G) * D + d] = __float2bfloat16_rn(acc / ll);
  }
  cluster_sync();                                    // every block has read: all may go
}

// The same end with the partials SENT instead of fetched, for requests whose partial is small (at most
// kPushRows packed rows and kPushFloats output elements: a decoded token of up to four query heads a kv
// head): every block stores each element of its partial into the inbox of the block that finishes that
// element, and its rows' maxima and sums into every block's inbox; after ONE cluster barrier every block
// finishes its share from its own shared memory and leaves.  Against cluster_finish this saves the trip of
// dependent loads through distributed shared memory after the barrier and the second barrier (nobody reads a
// block's memory after the barrier, so a block may leave at once).  `inbox` is shared memory that nothing
// else uses during the kernel — other blocks write it while this one is still working on its keys — of
// kPushInboxFloats floats.  Before the first store the caller has waited for the barrier at which every block
// of the cluster arrived when it started (cluster_started_*): a block's shared memory may be written by
// another only once it runs.
constexpr int kPushRows = 4;
constexpr int kPushFloats = 512;
constexpr int kPushInboxFloats = kPushFloats + kMaxCluster + kMaxCluster * kPushRows * 2;

__device__ __forceinline__ void cluster_started_arrive() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_started_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void store_to_cluster_block(float* local, uint32_t rank, float v) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(local));
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(a), "r"(rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

template <int D>
__device__ __forceinline__ void cluster_finish_push(const AttnParams& p, int g, int nsp, int packed, int G, int row0,
                                                    float (&m)[2], float (&l)[2], float (&o)[D / 8][4],
                                                    float* scratch, float* inbox) {
  constexpr int THREADS = 128;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
  }
  __syncthreads();                                   // the K/V tiles are no longer needed
  float* Ow = scratch;                               // [4][16][D]
  float* Mw = Ow + 4 * 16 * D;                       // [4][16]
  float* Lw = Mw + 4 * 16;                           // [4][16]
  float* In_o = inbox;                               // [nsp][share]: block c's partial of this block's elements
  float* In_ml = inbox + kPushFloats + kMaxCluster;  // [kMaxCluster][kPushRows][2]: block c's maximum and sum of every row
#pragma unroll
  for (int h = 0; h < 2 && warp < 4; ++h) {
    const int row = (lane >> 2) + h * 8;
    if (row >= packed) continue;
    float* orow = Ow + (warp * 16 + row) * D;
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      const int d = n * 8 + (lane & 3) * 2;
      *reinterpret_cast<float2*>(orow + d) = make_float2(o[n][2 * h], o[n][2 * h + 1]);
    }
    if ((lane & 3) == 0) {
      Mw[warp * 16 + row] = m[h];
      Lw[warp * 16 + row] = l[h];
    }
  }
  __syncthreads();
  const int total = packed * D;
  const int share = (total + nsp - 1) / nsp;
  const uint32_t me = cluster_rank();
  cluster_started_wait();                            // every block of the cluster runs: its inbox may be written
  for (int idx = threadIdx.x; idx < total && threadIdx.x < THREADS; idx += THREADS) {
    const int row = idx / D, d = idx % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, Mw[w * 16 + row]);
    float acc = 0.0f, ll = 0.0f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = Mw[w * 16 + row];
      if (mw == -INFINITY) continue;
      const float f = exp2f(mw - mm);
      acc += Ow[(w * 16 + row) * D + d] * f;
      ll += Lw[w * 16 + row] * f;
    }
    const int owner = idx / share;
    store_to_cluster_block(In_o + me * share + (idx - owner * share), owner, acc);
    if (d < nsp) {                                   // thread d of a row tells block d the row's maximum and sum
      store_to_cluster_block(In_ml + (me * kPushRows + row) * 2, d, mm);
      store_to_cluster_block(In_ml + (me * kPushRows + row) * 2 + 1, d, ll);
    }
  }
  cluster_sync();                                    // every block's stores have arrived
  const int first = static_cast<int>(me) * share;
  for (int idx = first + threadIdx.x; idx < min(total, first + share); idx += blockDim.x) {
    const int row = idx / D, d = idx % D;
    float pm[kMaxCluster], pl[kMaxCluster], po[kMaxCluster];
#pragma unroll
    for (int c = 0; c < kMaxCluster; ++c) {
      pm[c] = -INFINITY;
      pl[c] = po[c] = 0.0f;
      if (c < nsp) {
        pm[c] = In_ml[(c * kPushRows + row) * 2];
        pl[c] = In_ml[(c * kPushRows + row) * 2 + 1];
        po[c] = In_o[c * share + (idx - first)];
      }
    }
    float mm = -INFINITY;
#pragma unroll
    for (int c = 0; c < kMaxCluster; ++c) mm = fmaxf(mm, pm[c]);
    float acc = 0.0f, ll = 0.0f;
#pragma unroll
    for (int c = 0; c < kMaxCluster; ++c) {
      if (pm[c] == -INFINITY) continue;
      const float f = exp2f(pm[c] - mm);
      acc += po[c] * f;
      ll += pl[c] * f;
    }
    if (!(ll > 0.0f) || !isfinite(ll)) {
      publish_error(p.error, kAttentionDenominator);
      continue;
    }
    p.out[(static_cast<size_t>(row0 + row / G) * p.heads + g * G + row % G) * D + d] = __float2bfloat16_rn(acc / ll);
  }
}

constexpr int kSplitStages = 3;        // ring of K/V tiles in the split kernel

// Split kernel: 4 warps, at most 16 packed rows, grid (splits, kv_heads, R); decode-like requests.
// The tiles of a split stream through a ring of kSplitStages buffers (two tiles in flight while one is
// used), so a CTA keeps the memory system busy for the whole of its split.
template <int D>
__global__ void __launch_bounds__(128)
attn_split_kernel(const AttnParams p) {
  wait_for_prior_kernels();
  launch_dependents();                                   // (the next kernel's blocks may become resident and wait)
  constexpr int LD = D + 8;
  constexpr int THREADS = 128;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* KV = Qs + 16 * LD;                  // per stage: K [BN][LD] then V [BN][LD]
  __shared__ int s_last;

  const int r = blockIdx.z, g = blockIdx.y, sp = blockIdx.x;
  const int G = p.heads / p.kv_heads;
  const int row0 = p.cu_q[r];
  const int n_tok = p.cu_q[r + 1] - row0;
  const int packed = n_tok * G;
  if (packed > 16 || n_tok <= 0) return;             // the tile kernel's; a request of padding
  const int start = p.q_start[r];
  // keys that any row of the request sees, and the splits that hold them
  const int req_kmin = p.window > 0 ? max(0, start - p.window + 1) : 0;
  const int req_kmax = start + n_tok - 1;
  const int split = split_of(p);
  const int s_lo = req_kmin / split, s_hi = req_kmax / split;
  if (sp < s_lo || sp > s_hi) return;
  const int kmin = max(req_kmin, sp * split);
  const int kmax = min(req_kmax, (sp + 1) * split - 1);
  const int* table = p.block_table + static_cast<size_t>(r) * p.table_width;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  for (int c = threadIdx.x; c < 16 * (D / 8); c += THREADS) {
    const int row = c / (D / 8), ch = c % (D / 8);
    const bool valid = row < packed;
    const __nv_bfloat16* src = p.q;
    if (valid)
      src = p.q + static_cast<size_t>(row0 + row / G) * p.q_stride + static_cast<size_t>(g * G + row % G) * D + ch * 8;
    cp_async16(Qs + row * LD + ch * 8, src, valid ? 16 : 0);
  }
  const int t_first = kmin / BN, t_last = kmax / BN;
  const int ntiles = t_last - t_first + 1;
  for (int i = 0; i < kSplitStages - 1; ++i) {
    if (i < ntiles)
      load_kv_tile<D, THREADS>(p, table, g, (t_first + i) * BN, kmin, kmax, KV + (2 * i) * BN * LD,
                               KV + (2 * i + 1) * BN * LD);
    cp_async_commit();                               // one group per tile slot, empty or not
  }
  int row_pos[2], row_first[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int i = (lane >> 2) + h * 8;
    if (i < packed) {
      row_pos[h] = start + i / G;
      row_first[h] = p.window > 0 ? max(0, row_pos[h] - p.window + 1) : 0;
    } else {
      row_pos[h] = -1;
      row_first[h] = 0;
    }
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
  const float scale_log2 = p.scale * kLog2e;

  for (int i = 0; i < ntiles; ++i) {
    cp_async_wait<kSplitStages - 2>();               // tile i has landed
    __syncthreads();                                 // ... for everyone, and tile i - 1 is no longer read
    const int nxt = i + kSplitStages - 1;
    if (nxt < ntiles) {
      const int st = nxt % kSplitStages;
      load_kv_tile<D, THREADS>(p, table, g, (t_first + nxt) * BN, kmin, kmax, KV + (2 * st) * BN * LD,
                               KV + (2 * st + 1) * BN * LD);
    }
    cp_async_commit();
    // warp w takes keys 16 w .. 16 w + 15 of the tile
    const int st = i % kSplitStages;
    tile_step<D, 16, false>(Qs, KV + (2 * st) * BN * LD, KV + (2 * st + 1) * BN * LD, warp * 16,
                            (t_first + i) * BN + warp * 16, row_pos, row_first, scale_log2, m, l, o);
  }
  cp_async_wait<0>();
  split_finish<D>(p, r, g, sp, s_lo, s_hi, packed, G, row0, m, l, o, reinterpret_cast<float*>(KV), &s_last);
}

// Split kernel with TMA loads: the same work as attn_split_kernel, for head sizes that are multiples of 64
// and page sizes 8, 16, 32 or 64.  A fifth warp is the producer: one thread looks up the pages of a tile
// and issues one TMA box per (page, 64-column panel, K or V) with the 128-byte swizzle; the four consumer
// warps never compute an address.  Pages of a tile that hold no visible key are replaced by the first
// visible page, so that shared memory always holds finite values (they are masked by position).
// CLUSTER: the blocks of one (request, kv head) are one thread-block cluster (grid.x = cluster size = splits)
// and merge through distributed shared memory (cluster_finish) instead of scratch memory and tickets.
// FUSE: q arrives raw from the q/k/v product, with the new tokens' k and v beside it.  The consumer warps apply the
// per-head RMSNorm and the rotation to q on its way into shared memory; the block whose key range holds a new
// token's position does the same for that k, appends k and v to the cache and — because its TMA boxes may have
// read the cache before — puts them into the landed tile before it is used.  The q/k kernel between the q/k/v
// product and the attention is then not launched (2 us a layer at batch 8).
template <int D, bool CLUSTER, bool FUSE>
__global__ void __launch_bounds__(160)
attn_split_tma_kernel(const AttnParams p, const __grid_constant__ CUtensorMap kv_map) {
  // FUSE: what the block reads before its consumers wait for the kernel before this one — the step's batch arrays,
  // the block table, the cache's keys and values of earlier steps, norm weights, the rotation table — is written by
  // no kernel of this step, so the producer starts the stream of K/V tiles at once, while the q/k/v product is
  // still running; the consumers wait just before they read q and the new k and v.  (The new tokens' own keys,
  // which the boxes may bring in their old state, are put into the landed tile from registers anyway.)
  // Without FUSE the kernel before this one has written the new keys into the cache: everything waits for it.
  if (!FUSE) wait_for_prior_kernels();
  constexpr int LD = D + 8;
  constexpr int PANELS = D / 64;
  constexpr int TILE_BYTES = BN * D * 2;               // K (or V) of one tile: PANELS panels of BN x 128 bytes
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* KV = base;                            // per stage: K tile then V tile
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(base + kSplitStages * 2 * TILE_BYTES);
  uint64_t* full = reinterpret_cast<uint64_t*>(Qs + 16 * LD);
  uint64_t* empty = full + kSplitStages;
  __nv_bfloat16* NewK = reinterpret_cast<__nv_bfloat16*>(empty + kSplitStages);   // FUSE: [16][D], then NewV [16][D]
  __nv_bfloat16* NewV = NewK + 16 * D;
  __shared__ int s_last;

  const int r = blockIdx.z, g = blockIdx.y, sp = blockIdx.x;
  const int G = p.heads / p.kv_heads;
  const int row0 = p.cu_q[r];
  const int n_tok = p.cu_q[r + 1] - row0;
  const int packed = n_tok * G;
  if (packed > 16 || n_tok <= 0) return;               // the tile kernel's; a request of padding (a whole cluster leaves)
  const int start = p.q_start[r];
  const int req_kmin = p.window > 0 ? max(0, start - p.window + 1) : 0;
  const int req_kmax = start + n_tok - 1;
  const int split = split_of(p);
  const int s_lo = req_kmin / split, s_hi = req_kmax / split;
  const bool has_keys = sp >= s_lo && sp <= s_hi;
  if (!CLUSTER && !has_keys) return;                   // (in a cluster every block stays for the barriers)
  const int kmin = max(req_kmin, sp * split);
  const int kmax = min(req_kmax, (sp + 1) * split - 1);
  const int* table = p.block_table + static_cast<size_t>(r) * p.table_width;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t_first = kmin / BN, t_last = kmax / BN;
  const int ntiles = has_keys ? t_last - t_first + 1 : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kSplitStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 4);                         // one arrival per consumer warp
    }
    mbar_init_fence();
  }
  __syncthreads();                                     // barriers initialised
  if (CLUSTER && p.push_merge) cluster_started_arrive();   // waited for before the first store into another block

  int row_pos[2], row_first[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int i = (lane >> 2) + h * 8;
    if (i < packed) {
      row_pos[h] = start + i / G;
      row_first[h] = p.window > 0 ? max(0, row_pos[h] - p.window + 1) : 0;
    } else {
      row_pos[h] = -1;
      row_first[h] = 0;
    }
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
  const float scale_log2 = p.scale * kLog2e;

  if (warp == 4) {
    // producer: lane pg looks up page pg of the tile and issues its boxes; lane 0 announces the bytes
    const int pages_per_tile = BN >> p.page_shift;
    const int fallback = kmin >> p.page_shift;          // a page that certainly exists
    if (lane == 0) tma_prefetch_map(&kv_map);
    bool alive = true;
    for (int i = 0; i < ntiles && alive; ++i) {
      const int s = i % kSplitStages;
      const int round = i / kSplitStages;
      int page = 0;
      if (lane < pages_per_tile) {                      // the look-up overlaps the wait for the buffer
        const int j_page = (t_first + i) * BN + lane * p.page_size;
        const bool seen = j_page <= kmax && j_page + p.page_size - 1 >= kmin;
        page = table[seen ? (j_page >> p.page_shift) : fallback];
        if (page < 0 || page >= p.num_pages) {
          publish_error(p.error, kRowWithoutPage);
          page = 0;
        }
      }
      if (round > 0) alive = mbar_wait(&empty[s], (round - 1) & 1, p.error);
      alive = __all_sync(0xffffffffu, alive);
      if (!alive) break;
      if (lane == 0) mbar_expect_tx(&full[s], 2 * TILE_BYTES);
      __syncwarp();
      if (lane < pages_per_tile) {
        unsigned char* kdst = KV + s * 2 * TILE_BYTES + lane * p.page_size * 128;
        unsigned char* vdst = kdst + TILE_BYTES;
        const int zk = (page * 2) * p.kv_heads + g, zv = (page * 2 + 1) * p.kv_heads + g;
#pragma unroll
        for (int pn = 0; pn < PANELS; ++pn) {
          tma_load_3d(kdst + pn * (BN * 128), &kv_map, pn * 64, 0, zk, &full[s]);
          tma_load_3d(vdst + pn * (BN * 128), &kv_map, pn * 64, 0, zv, &full[s]);
        }
      }
    }
    // the block's last load is on its way: once every block says so, the next kernel's blocks may become resident
    // and start streaming their weights
    if (lane == 0) launch_dependents();
  } else {
    // consumers: the query rows arrive while the first tiles are on their way
    if (FUSE) {
      constexpr int EPL = D / 32;
      constexpr int HALF = D / 2;
      struct alignas(EPL * 2) Pack { __nv_bfloat16 e[EPL]; };
      auto weights = [&](const void* w, float (&out)[EPL]) {
#pragma unroll
        for (int j = 0; j < EPL; ++j)
          out[j] = p.norm_w_f32 ? static_cast<const float*>(w)[lane * EPL + j]
                                : __bfloat162float(static_cast<const __nv_bfloat16*>(w)[lane * EPL + j]);
      };
      auto angles = [&](int pos, float2 (&cs)[EPL]) {
        if (pos < 0 || pos >= p.max_pos) {
          if (lane == 0) publish_error(p.error, kBadPosition);
          pos = 0;
        }
        const float2* src = reinterpret_cast<const float2*>(p.rope) + static_cast<size_t>(pos) * HALF + (lane & 15) * EPL;
#pragma unroll
        for (int j = 0; j < EPL; ++j) cs[j] = src[j];
      };
      float wq[EPL], wk[EPL];
      if (p.q_norm_w != nullptr) weights(p.q_norm_w, wq);
      if (p.k_norm_w != nullptr) weights(p.k_norm_w, wk);
      // The block's tasks: its query rows, then the new tokens whose positions lie in its key range (their k is
      // normed and rotated, their v kept, both appended to the cache and held for the tile that the TMA boxes may
      // have filled from the cache's old contents).  Task t goes to warp t % 4, so the tasks' loads — one trip to
      // the L2 each — run side by side; rows beyond the request's are zero.  The first task's rotation angles
      // depend on the position alone: they are fetched before the wait.
      const int nk = (p.write_kv && has_keys) ? n_tok : 0;
      const int ntasks = packed + nk;
      auto position_of = [&](int t) { return t < packed ? start + t / G : start + (t - packed); };
      for (int row = packed + warp; row < 16; row += 4) {
        Pack zero;
#pragma unroll
        for (int j = 0; j < EPL; ++j) zero.e[j] = __float2bfloat16_rn(0.0f);
        *reinterpret_cast<Pack*>(Qs + row * LD + lane * EPL) = zero;
      }
      float2 cs_first[EPL];
      if (p.rope != nullptr && warp < ntasks) angles(position_of(warp), cs_first);
      wait_for_prior_kernels();                            // q and the new k and v are the kernel before's output
      for (int t = warp; t < ntasks; t += 4) {
        const bool is_q = t < packed;
        const int tt = is_q ? t / G : t - packed;          // the token of the step
        const int j = start + tt;                          // its position
        if (!is_q && (j < kmin || j > kmax)) continue;
        const __nv_bfloat16* src = p.q + static_cast<size_t>(row0 + tt) * p.q_stride +
                                   static_cast<size_t>(is_q ? g * G + t % G : p.heads + g) * D + lane * EPL;
        const Pack in = *reinterpret_cast<const Pack*>(src);
        Pack vin;
        if (!is_q) vin = *reinterpret_cast<const Pack*>(src + static_cast<size_t>(p.kv_heads) * D);
        float v[EPL];
        float2 cs[EPL];
#pragma unroll
        for (int e = 0; e < EPL; ++e) v[e] = __bfloat162float(in.e[e]);
        if (p.rope != nullptr) {
          if (t == warp) {
#pragma unroll
            for (int e = 0; e < EPL; ++e) cs[e] = cs_first[e];
          } else {
            angles(j, cs);
          }
        }
        const void* nw = is_q ? p.q_norm_w : p.k_norm_w;
        head_norm_rotate<__nv_bfloat16, float, EPL>(v, nw != nullptr ? (is_q ? wq : wk) : nullptr, p.norm_eps,
                                                    p.rope != nullptr ? cs : nullptr, lane);
        Pack outp;
#pragma unroll
        for (int e = 0; e < EPL; ++e) outp.e[e] = __float2bfloat16_rn(v[e]);
        if (is_q) {
          *reinterpret_cast<Pack*>(Qs + t * LD + lane * EPL) = outp;
          continue;
        }
        int page = table[j >> p.page_shift];
        if (page < 0 || page >= p.num_pages) {
          if (lane == 0) publish_error(p.error, kRowWithoutPage);
        } else {
          __nv_bfloat16* dst = p.cache_w + (static_cast<size_t>(page) * 2 * p.kv_heads + g) * p.page_size * D +
                               static_cast<size_t>(j & (p.page_size - 1)) * D + lane * EPL;
          *reinterpret_cast<Pack*>(dst) = outp;
          *reinterpret_cast<Pack*>(dst + static_cast<size_t>(p.kv_heads) * p.page_size * D) = vin;
        }
        *reinterpret_cast<Pack*>(NewK + tt * D + lane * EPL) = outp;
        *reinterpret_cast<Pack*>(NewV + tt * D + lane * EPL) = vin;
      }
    } else {
      for (int c = threadIdx.x; c < 16 * (D / 8); c += 128) {
        const int row = c / (D / 8), ch = c % (D / 8);
        const bool valid = row < packed;
        const __nv_bfloat16* src = p.q;
        if (valid)
          src = p.q + static_cast<size_t>(row0 + row / G) * p.q_stride + static_cast<size_t>(g * G + row % G) * D + ch * 8;
        cp_async16(Qs + row * LD + ch * 8, src, valid ? 16 : 0);
      }
      cp_async_commit();
      cp_async_wait<0>();
    }
    asm volatile("bar.sync 1, 128;\n" ::: "memory");   // the four consumer warps only
    for (int i = 0; i < ntiles; ++i) {
      const int s = i % kSplitStages;
      mbar_wait(&full[s], (i / kSplitStages) & 1, p.error);
      const __nv_bfloat16* Ks = reinterpret_cast<const __nv_bfloat16*>(KV + s * 2 * TILE_BYTES);
      const __nv_bfloat16* Vs = reinterpret_cast<const __nv_bfloat16*>(KV + s * 2 * TILE_BYTES + TILE_BYTES);
      if (FUSE && p.write_kv) {
        // new tokens among this warp's 16 keys of the tile: their k and v replace what the boxes brought
        constexpr int EPL = D / 32;
        struct alignas(EPL * 2) Pack { __nv_bfloat16 e[EPL]; };
        const int tile_j0 = (t_first + i) * BN;
        const int lo = max(tile_j0 + warp * 16, max(start, kmin));
        const int hi = min(tile_j0 + warp * 16 + 15, min(start + n_tok - 1, kmax));
        for (int j = lo; j <= hi; ++j) {
          const int tt = j - start, rr = j - tile_j0;
          const int col = lane * EPL;                      // kv_at gives the 16-byte chunk; the lane's place inside it
          *reinterpret_cast<Pack*>(const_cast<__nv_bfloat16*>(kv_at<D, true>(Ks, rr, col & ~7)) + (col & 7)) =
              *reinterpret_cast<const Pack*>(NewK + tt * D + col);
          *reinterpret_cast<Pack*>(const_cast<__nv_bfloat16*>(kv_at<D, true>(Vs, rr, col & ~7)) + (col & 7)) =
              *reinterpret_cast<const Pack*>(NewV + tt * D + col);
        }
        __syncwarp();
      }
      tile_step<D, 16, true>(Qs, Ks, Vs, warp * 16, (t_first + i) * BN + warp * 16, row_pos, row_first, scale_log2,
                             m, l, o);
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
    }
  }
  __syncwarp();
  if (CLUSTER && p.push_merge)
    cluster_finish_push<D>(p, g, static_cast<int>(gridDim.x), packed, G, row0, m, l, o, reinterpret_cast<float*>(KV),
                           reinterpret_cast<float*>(NewV + 16 * D));
  else if (CLUSTER)
    cluster_finish<D>(p, g, static_cast<int>(gridDim.x), packed, G, row0, m, l, o, reinterpret_cast<float*>(KV));
  else
    split_finish<D>(p, r, g, sp, s_lo, s_hi, packed, G, row0, m, l, o, reinterpret_cast<float*>(KV), &s_last);
}

// 1: the splits of one (request, kv head) are a thread-block cluster when there are 2 to kMaxCluster of them
int g_cluster_merge = 1;


template <int D>
static int launch_split_tma(const AttnParams& params, int R, const CUtensorMap* kv_map, cudaStream_t s) {
  if constexpr (D % 64 == 0) {
    constexpr int LD = D + 8;
    AttnParams p = params;
    const bool cluster = g_cluster_merge && p.max_splits >= 2 && p.max_splits <= kMaxCluster;
    int smem = 1024 + kSplitStages * 2 * BN * D * 2 + 16 * LD * 2 + 2 * kSplitStages * 8 + 2 * 16 * D * 2;
    const int merge = 1024 + (4 * 16 * D + 128 + 16 * D + 32 + 32 * p.max_splits + 16) * 4;
    if (merge > smem) smem = merge;
    // small partials are sent to the blocks that finish them (cluster_finish_push): the inbox lies behind all else
    const int packed_cap = p.dec_tok_cap * (p.heads / p.kv_heads);
    p.push_merge = cluster && g_cluster_merge == 1 && packed_cap <= kPushRows && packed_cap * D <= kPushFloats;
    if (p.push_merge) smem += kPushInboxFloats * 4;
    if (smem > 227 * 1024) return PIH_ERR_UNSUPPORTED;
    dim3 grid(p.max_splits, p.kv_heads, R);
#define PIH_SPLIT_TMA(CLUSTER, FUSE)                                                                              \
  do {                                                                                                            \
    static int smem_done = -1;                                                                                    \
    if (smem_done < 0) {                                                                                          \
      /* the same preference as the products of a decode step: their blocks may then be resident beside these */  \
      cudaError_t e = cudaFuncSetAttribute(attn_split_tma_kernel<D, CLUSTER, FUSE>,                               \
                                           cudaFuncAttributePreferredSharedMemoryCarveout,                        \
                                           cudaSharedmemCarveoutMaxShared);                                       \
      if (e != cudaSuccess) return static_cast<int>(e);                                                           \
      smem_done = 0;                                                                                              \
    }                                                                                                             \
    if (smem_done < smem) {                                                                                       \
      cudaError_t e = cudaFuncSetAttribute(attn_split_tma_kernel<D, CLUSTER, FUSE>,                               \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, smem);                    \
      if (e != cudaSuccess) return static_cast<int>(e);                                                           \
      smem_done = smem;                                                                                           \
    }                                                                                                             \
    launch_kernel_clustered(attn_split_tma_kernel<D, CLUSTER, FUSE>, grid, dim3(160), smem, s,                    \
                            CLUSTER ? static_cast<unsigned>(p.max_splits) : 1u, p, *kv_map);                      \
  } while (0)
    if (cluster && p.fused) PIH_SPLIT_TMA(true, true);
    else if (cluster) PIH_SPLIT_TMA(true, false);
    else if (p.fused) PIH_SPLIT_TMA(false, true);
    else PIH_SPLIT_TMA(false, false);
#undef PIH_SPLIT_TMA
    PIH_LAUNCH_CHECK();
    return 0;
  } else {
    return PIH_ERR_UNSUPPORTED;
  }
}

template <int D>
static int launch_both(const AttnParams& p, int R, int tile_max_q, const CUtensorMap* kv_map, cudaStream_t s) {
  constexpr int LD = D + 8;
  const int G = p.heads / p.kv_heads;
  static int tile_smem_set = 0, split_smem_set = 0;   // per head_dim instance
  if (tile_max_q > 0) {
    const int smem = (64 * LD + 4 * BN * LD) * static_cast<int>(sizeof(__nv_bfloat16));
    if (tile_smem_set < smem) {
      cudaError_t e = cudaFuncSetAttribute(attn_tile_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return static_cast<int>(e);
      tile_smem_set = smem;
    }
    dim3 grid((tile_max_q * G + 63) / 64, p.kv_heads, R);
    launch_kernel(attn_tile_kernel<D>, dim3(grid), dim3(128), smem, s, p);
    PIH_LAUNCH_CHECK();
  }
  if (p.dec_tok_cap > 0 && kv_map != nullptr && D % 64 == 0 && p.page_shift >= 3 && p.page_size <= BN) {
    return launch_split_tma<D>(p, R, kv_map, s);
  }
  if (p.dec_tok_cap > 0) {
    int smem = (16 * LD + 2 * kSplitStages * BN * LD) * static_cast<int>(sizeof(__nv_bfloat16));
    const int merge = 16 * LD * static_cast<int>(sizeof(__nv_bfloat16)) + (4 * 16 * D + 128) * static_cast<int>(sizeof(float));
    if (merge > smem) smem = merge;
    const int final_merge = 16 * LD * static_cast<int>(sizeof(__nv_bfloat16)) +
                            (32 * p.max_splits + 16) * static_cast<int>(sizeof(float));
    if (final_merge > smem) smem = final_merge;
    if (smem > 227 * 1024) return PIH_ERR_UNSUPPORTED;
    if (split_smem_set < smem) {
      cudaError_t e = cudaFuncSetAttribute(attn_split_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return static_cast<int>(e);
      split_smem_set = smem;
    }
    dim3 grid(p.max_splits, p.kv_heads, R);
    launch_kernel(attn_split_kernel<D>, dim3(grid), dim3(128), smem, s, p);
    PIH_LAUNCH_CHECK();
  }
  return 0;
}

}  // namespace pih

using namespace pih;

// 1 (the default): 2 to 8 splits of one (request, kv head) run as a thread-block cluster and merge through
// distributed shared memory, small partials sent and larger ones fetched; 2: always fetched; 0: every split
// count merges through scratch memory and tickets.  Returns the previous setting.
extern "C" int pih_set_attention_cluster_merge(int mode) {
  const int before = pih::g_cluster_merge;
  pih::g_cluster_merge = mode < 0 ? 0 : mode > 2 ? 2 : mode;
  return before;
}

// Floats (4-byte words) of scratch that the split kernel needs: tickets first, then the partials.
// The first pih_attention_ticket_words(...) words must be zero before the first launch; the kernel
// leaves them zero.
extern "C" long long pih_attention_ticket_words(int num_requests, int kv_heads) {
  return (static_cast<long long>(num_requests) * kv_heads + 63) / 64 * 64;
}
extern "C" long long pih_attention_scratch_floats(int num_requests, int dec_tok_cap, int heads, int kv_heads,
                                                  int head_dim, int max_splits) {
  return pih_attention_ticket_words(num_requests, kv_heads) +
         static_cast<long long>(num_requests) * dec_tok_cap * heads * max_splits * (head_dim + 2);
}

// Describes one schedule entry's cache [num_pages, 2, kv_heads, page_size, head_dim] (bf16) to TMA as a
// 3-D tensor (head_dim, page_size, num_pages * 2 * kv_heads) with boxes of 64 columns x one page and the
// 128-byte swizzle.  `out` receives 128 bytes.  PIH_ERR_UNSUPPORTED when the shape has no such form.
extern "C" int pih_make_kv_tensor_map(void* out, const void* cache, long long num_pages, int kv_heads,
                                      int page_size, int head_dim) {
  if (head_dim % 64 || page_size < 8 || page_size > 256 || (page_size & (page_size - 1)) ||
      (reinterpret_cast<uintptr_t>(cache) & 15))
    return PIH_ERR_UNSUPPORTED;
  EncodeTiledFn fn = encode_tiled();
  if (fn == nullptr) return PIH_ERR_UNSUPPORTED;
  CUtensorMap map;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(page_size),
                              static_cast<cuuint64_t>(num_pages) * 2 * kv_heads};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(head_dim) * 2,
                                 static_cast<cuuint64_t>(page_size) * head_dim * 2};
  const cuuint32_t box[3] = {64, static_cast<cuuint32_t>(page_size < BN ? page_size : BN), 1};
  const cuuint32_t elem[3] = {1, 1, 1};
  if (fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(cache), dims, strides, box, elem,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return PIH_ERR_UNSUPPORTED;
  memcpy(out, &map, sizeof(CUtensorMap));
  return 0;
}

// A request is "decode-like" when it brings at most 16 packed rows (rows * heads / kv_heads <= 16).
//   tile_max_q   the most rows of a request that is NOT decode-like (0: there is none)
//   dec_tok_cap  the most rows of a decode-like request (0: there is none)
//   dec_max_ctx  the longest context (after the step) of a decode-like request
//   split        keys per split; or 0 with max_splits > 0 and max_ctx_ptr a device word holding the step's longest
//                context: each request is then cut into max_splits parts of that context
// scratch holds pih_attention_scratch_floats(num_requests, dec_tok_cap, heads, kv_heads, head_dim,
// ceil(dec_max_ctx / split)) words, the leading ticket words zero.  Launches that share the scratch
// must not overlap on the device.  Returns PIH_ERR_UNSUPPORTED for a head_dim that has no
// tensor-core instance (the caller then uses the generic kernel).
namespace pih {
struct QkFusion {                      // what the split kernel needs to norm and rotate q and k itself
  const void* q_norm_w;
  const void* k_norm_w;
  int norm_w_f32;
  float eps;
  const float* rope;
  int max_pos;
  int write_kv;
};
}  // namespace pih

static int paged_attention_mma(const void* q, int q_stride, void* out, const void* cache,
                               const int* block_table, int table_width, const int* cu_q,
                               const int* q_start, int rows, int num_requests, int tile_max_q,
                               int dec_tok_cap, int dec_max_ctx, int heads, int kv_heads, int head_dim,
                               int page_size, int num_pages, float scale, int window, int split,
                               int max_splits, const int* max_ctx_ptr, float* scratch,
                               const void* kv_tensor_map, uint32_t* error, void* stream, const QkFusion* fusion) {
  if (rows <= 0) return 0;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || page_size <= 0 || table_width <= 0 || window < 0 ||
      split < 0 || split % BN || (split == 0 && dec_tok_cap > 0 && (max_splits <= 0 || max_ctx_ptr == nullptr)) ||
      num_requests <= 0 || num_requests > 65535 ||
      kv_heads > 65535 || q_stride % 8 || tile_max_q < 0 || dec_tok_cap < 0 ||
      (dec_tok_cap > 0 && (dec_max_ctx <= 0 || !scratch || (reinterpret_cast<uintptr_t>(scratch) & 7))))
    return PIH_ERR_BAD_ARGUMENT;   // (the merge reads a split's maximum and sum as one 8-byte word)
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
  p.max_ctx_ptr = max_ctx_ptr;
  p.max_splits = dec_tok_cap == 0 ? 0 : (split > 0 ? (dec_max_ctx + split - 1) / split : max_splits);
  p.dec_tok_cap = dec_tok_cap;
  p.page_shift = -1;
  for (int sft = 0; sft < 20; ++sft)
    if ((1 << sft) == page_size) p.page_shift = sft;
  const long long tickets = pih_attention_ticket_words(num_requests, kv_heads);
  p.tickets = reinterpret_cast<int*>(scratch);
  p.part_o = scratch + tickets;
  p.part_ml = p.part_o + static_cast<size_t>(num_requests) * dec_tok_cap * heads * p.max_splits * head_dim;
  p.error = error;
  p.fused = 0;
  p.q_norm_w = p.k_norm_w = nullptr;
  p.rope = nullptr;
  p.norm_w_f32 = p.max_pos = p.write_kv = 0;
  p.norm_eps = 0.0f;
  p.cache_w = nullptr;
  if (fusion != nullptr) {
    // only the TMA split kernel does the q/k work itself: every request decode-like, a head on 32 lanes
    if (tile_max_q > 0 || dec_tok_cap <= 0 || kv_tensor_map == nullptr || head_dim % 64 || p.page_shift < 3 ||
        page_size > BN || (fusion->rope != nullptr && fusion->max_pos <= 0))
      return PIH_ERR_UNSUPPORTED;
    p.fused = 1;
    p.q_norm_w = fusion->q_norm_w;
    p.k_norm_w = fusion->k_norm_w;
    p.norm_w_f32 = fusion->norm_w_f32;
    p.norm_eps = fusion->eps;
    p.rope = fusion->rope;
    p.max_pos = fusion->max_pos;
    p.write_kv = fusion->write_kv;
    p.cache_w = static_cast<__nv_bfloat16*>(const_cast<void*>(cache));
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  CUtensorMap map_storage;
  const CUtensorMap* kv_map = nullptr;
  if (kv_tensor_map != nullptr) {
    memcpy(&map_storage, kv_tensor_map, sizeof(CUtensorMap));
    kv_map = &map_storage;
  }
  switch (head_dim) {
    case 16: return launch_both<16>(p, num_requests, tile_max_q, kv_map, s);
    case 32: return launch_both<32>(p, num_requests, tile_max_q, kv_map, s);
    case 64: return launch_both<64>(p, num_requests, tile_max_q, kv_map, s);
    case 80: return launch_both<80>(p, num_requests, tile_max_q, kv_map, s);
    case 96: return launch_both<96>(p, num_requests, tile_max_q, kv_map, s);
    case 128: return launch_both<128>(p, num_requests, tile_max_q, kv_map, s);
    case 256: return launch_both<256>(p, num_requests, tile_max_q, kv_map, s);
    default: return PIH_ERR_UNSUPPORTED;
  }
}

extern "C" int pih_paged_attention_mma(const void* q, int q_stride, void* out, const void* cache,
                                       const int* block_table, int table_width, const int* cu_q,
                                       const int* q_start, int rows, int num_requests, int tile_max_q,
                                       int dec_tok_cap, int dec_max_ctx, int heads, int kv_heads, int head_dim,
                                       int page_size, int num_pages, float scale, int window, int split,
                                       int max_splits, const int* max_ctx_ptr, float* scratch,
                                       const void* kv_tensor_map, uint32_t* error, void* stream) {
  return paged_attention_mma(q, q_stride, out, cache, block_table, table_width, cu_q, q_start, rows, num_requests,
                             tile_max_q, dec_tok_cap, dec_max_ctx, heads, kv_heads, head_dim, page_size, num_pages,
                             scale, window, split, max_splits, max_ctx_ptr, scratch, kv_tensor_map, error, stream,
                             nullptr);
}

// Decode attention that also does what pih_qk_norm_rope_kv_write does: qkv holds the raw rows [q | k | v] of the
// q/k/v product (row stride q_stride); q and the new tokens' k get the per-head RMSNorm (weights q_norm_w, k_norm_w
// of dtype norm_dtype, nullable) and the rotation (rope [max_pos, head_dim / 2, 2], nullable, over the whole head),
// and with write_kv the new k and v are appended to the cache.  qkv itself is left as it is.  For steps whose
// requests are all decode-like and shapes that the TMA split kernel takes; PIH_ERR_UNSUPPORTED otherwise, with
// nothing launched (the caller runs the two kernels).
extern "C" int pih_qk_attention_fused(const void* qkv, int q_stride, void* out, void* cache, const int* block_table,
                                      int table_width, const int* cu_q, const int* q_start, int rows, int num_requests,
                                      int dec_tok_cap, int dec_max_ctx, int heads, int kv_heads, int head_dim,
                                      int page_size, int num_pages, float scale, int window, int split, int max_splits,
                                      const int* max_ctx_ptr, float* scratch, const void* kv_tensor_map,
                                      int norm_dtype, const void* q_norm_w, const void* k_norm_w, float eps,
                                      const float* rope, int max_pos, int write_kv, uint32_t* error, void* stream) {
  if (norm_dtype != PIH_BF16 && norm_dtype != PIH_F32) return PIH_ERR_BAD_ARGUMENT;
  QkFusion f = {q_norm_w, k_norm_w, norm_dtype == PIH_F32 ? 1 : 0, eps, rope, max_pos, write_kv};
  return paged_attention_mma(qkv, q_stride, out, cache, block_table, table_width, cu_q, q_start, rows, num_requests, 0,
                             dec_tok_cap, dec_max_ctx, heads, kv_heads, head_dim, page_size, num_pages, scale, window,
                             split, max_splits, max_ctx_ptr, scratch, kv_tensor_map, error, stream, &f);
}
