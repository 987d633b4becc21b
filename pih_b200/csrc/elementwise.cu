// Memory-bound ops of the step: embedding gather, (residual add +) RMSNorm,
// per-head q/k RMSNorm + RoPE + cache write, SiLU-mul.  Every kernel is a
// template over the storage type (float for the true 32-bit path,
// __nv_bfloat16 for serving) and takes every size as an argument.
#include "common.cuh"
#include "qk_math.cuh"

namespace pih {

// ---------------------------------------------------------------------------
// embedding: out[t,:] = table[ids[t],:]    (reference: qwen_bf16_primitives.cu:247-262,
// which skips ids outside the table silently; here they are reported)
// ---------------------------------------------------------------------------
template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                 T* __restrict__ out, int rows, int hidden, int vocab,
                                 uint32_t* error) {
  wait_for_prior_kernels();
  launch_dependents();                                   // (the next kernel's blocks may become resident and wait)
  const int t = blockIdx.x;
  if (t >= rows) return;
  int id = ids[t];
  const bool bad = id < 0 || id >= vocab;
  if (bad) {
    if (threadIdx.x == 0) publish_error(error, kTokenOutOfVocabulary);
    id = 0;
  }
  const T* src = table + static_cast<size_t>(id) * hidden;
  T* dst = out + static_cast<size_t>(t) * hidden;
  const int row_bytes = hidden * static_cast<int>(sizeof(T));
  if (row_bytes % 16 == 0) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    for (int i = threadIdx.x; i < row_bytes / 16; i += blockDim.x)
      d4[i] = bad ? make_uint4(0, 0, 0, 0) : s4[i];
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
      dst[i] = bad ? from_float<T>(0.0f) : src[i];
  }
}

// ---------------------------------------------------------------------------
// (residual add +) RMSNorm, one block per output row.
//   in place (rows == nullptr): x[r] = round(x[r] + delta[r]) is stored back and normed
//   gathered (rows != nullptr): out[i] = norm(round(x[rows[i]] + delta[rows[i]])), x untouched
// y = round( (v * 1/sqrt(mean(v^2) + eps)) * w )      (qwen_bf16_primitives.cu:285-324)
// ---------------------------------------------------------------------------
template <typename T, typename W>
__global__ void rmsnorm_kernel(T* __restrict__ x, const T* __restrict__ delta,
                               const W* __restrict__ weight, T* __restrict__ out,
                               const int* __restrict__ rows, int width, float eps) {
  wait_for_prior_kernels();
  launch_dependents();                                   // (the next kernel's blocks may become resident and wait)
  __shared__ float scratch[33];
  const int o = blockIdx.x;
  const size_t r = rows != nullptr ? static_cast<size_t>(rows[o]) : static_cast<size_t>(o);
  T* xr = x + r * width;
  const T* dr = delta != nullptr ? delta + r * width : nullptr;
  const bool write_back = delta != nullptr && rows == nullptr;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = to_float<T>(xr[c]);
    if (dr != nullptr) {
      v = round_to<T>(v + to_float<T>(dr[c]));
      if (write_back) xr[c] = from_float<T>(v);
    }
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / static_cast<float>(width) + eps);
  T* yr = out + static_cast<size_t>(o) * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = to_float<T>(xr[c]);                      // after write_back this is the rounded sum
    if (dr != nullptr && !write_back) v = round_to<T>(v + to_float<T>(dr[c]));
    yr[c] = from_float<T>((v * scale) * to_float<W>(weight[c]));
  }
}

// ---------------------------------------------------------------------------
// Per-head RMSNorm of q and k, rotate-half RoPE from a (cos, sin) table, and the
// write of k and v into the paged cache: one warp per (row, head slot).
//   slot <  heads                      : q head, normed and rotated in place
//   slot <  heads + kv_heads           : k head, normed, rotated, stored in place and in the cache
//   slot <  heads + 2 kv_heads         : v head, copied into the cache
// Rounding as the reference's separate kernels give it: once after the norm,
// once after the rotation (qwen_bf16_primitives.cu:285-347), cache write is a copy (:468-517).
// cache layout: [page][2][kv_head][page_size][head_dim]
// ---------------------------------------------------------------------------
template <typename T, typename W>
__global__ void qk_norm_rope_kv_kernel(T* __restrict__ qkv, int row_stride, int rows, int heads,
                                       int kv_heads, int head_dim, const W* __restrict__ q_w,
                                       const W* __restrict__ k_w, float eps,
                                       const float* __restrict__ rope, int rotary_dim, int max_pos,
                                       const int* __restrict__ positions,
                                       const int* __restrict__ slot_mapping, T* __restrict__ cache,
                                       int page_size, int num_pages, int write_kv, uint32_t* error) {
  wait_for_prior_kernels();
  launch_dependents();                                   // (the next kernel's blocks may become resident and wait)
  extern __shared__ float smem[];
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slots = heads + (write_kv ? 2 * kv_heads : 0);
  const long long item = static_cast<long long>(blockIdx.x) * warps_per_block + warp;
  if (item >= static_cast<long long>(rows) * slots) return;
  const int t = static_cast<int>(item / slots);
  const int slot = static_cast<int>(item % slots);
  float* buf = smem + warp * head_dim;
  T* src = qkv + static_cast<size_t>(t) * row_stride + static_cast<size_t>(slot) * head_dim;

  const bool is_q = slot < heads;
  const bool is_k = !is_q && slot < heads + kv_heads;
  const bool is_v = !is_q && !is_k;
  T* dst_cache = nullptr;
  if (!is_q) {
    const int m = slot_mapping[t];
    if (m < 0 || m >= num_pages * page_size) {
      if (lane == 0 && m != kPaddingSlot) publish_error(error, kRowWithoutPage);   // (a row of padding is left alone)
    } else {
      const int page = m / page_size, off = m % page_size;
      const int h = is_k ? slot - heads : slot - heads - kv_heads;
      dst_cache = cache + ((static_cast<size_t>(page) * 2 + (is_k ? 0 : 1)) * kv_heads + h) *
                              page_size * head_dim + static_cast<size_t>(off) * head_dim;
    }
  }
  if (is_v) {
    if (dst_cache != nullptr)
      for (int c = lane; c < head_dim; c += 32) dst_cache[c] = src[c];
    return;
  }
  const W* w = is_q ? q_w : k_w;
  // norm
  float ss = 0.0f;
  for (int c = lane; c < head_dim; c += 32) {
    const float v = to_float<T>(src[c]);
    buf[c] = v;
    ss += v * v;
  }
  if (w != nullptr) {
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / static_cast<float>(head_dim) + eps);
    for (int c = lane; c < head_dim; c += 32)
      buf[c] = round_to<T>((buf[c] * scale) * to_float<W>(w[c]));
  }
  __syncwarp();
  // rotation
  const int half = rotary_dim / 2;
  int pos = positions[t];
  if (rope != nullptr && (pos < 0 || pos >= max_pos)) {
    if (lane == 0) publish_error(error, kBadPosition);
    pos = 0;
  }
  const float* cs = rope != nullptr ? rope + static_cast<size_t>(pos) * half * 2 : nullptr;
  for (int c = lane; c < head_dim; c += 32) {
    float v = buf[c];
    if (cs != nullptr && c < rotary_dim) {
      if (c < half) {
        v = buf[c] * cs[2 * c] - buf[c + half] * cs[2 * c + 1];
      } else {
        const int p = c - half;
        v = buf[c] * cs[2 * p] + buf[p] * cs[2 * p + 1];
      }
    }
    const T r = from_float<T>(v);
    src[c] = r;
    if (dst_cache != nullptr) dst_cache[c] = r;
  }
}

// Fast path of the kernel above for head_dim = 32 * EPL with EPL in {2, 4, 8} and a rotation over
// the whole head: a lane keeps EPL contiguous elements in registers; its rotation partner (i +- D/2)
// sits in lane ^ 16.  Same arithmetic and roundings as the general kernel.
// A warp takes SPW consecutive head slots (q heads, then k heads, then v heads) of one row: their loads are
// issued together, and what depends on the row alone — position, cache slot, the lane's cosines and sines —
// is fetched once for all of them, as 16-byte loads.  (One slot per warp with scalar loads of weights and
// angles was bound by instruction issue: 22 us for 2048 rows of 16 + 8 + 8 heads of 128.)
template <typename T, typename W, int EPL, int SPW>
__global__ void qk_norm_rope_kv_fast_kernel(T* __restrict__ qkv, int row_stride, int rows, int heads,
                                            int kv_heads, const W* __restrict__ q_w,
                                            const W* __restrict__ k_w, float eps,
                                            const float* __restrict__ rope, int max_pos,
                                            const int* __restrict__ positions,
                                            const int* __restrict__ slot_mapping, T* __restrict__ cache,
                                            int page_size, int num_pages, int write_kv, uint32_t* error) {
  wait_for_prior_kernels();
  launch_dependents();                                   // (the next kernel's blocks may become resident and wait)
  constexpr int D = 32 * EPL;
  constexpr int HALF = D / 2;
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slots = heads + (write_kv ? 2 * kv_heads : 0);
  const int groups = (slots + SPW - 1) / SPW;
  const long long item = static_cast<long long>(blockIdx.x) * warps_per_block + warp;
  if (item >= static_cast<long long>(rows) * groups) return;
  const int t = static_cast<int>(item / groups);
  const int slot0 = static_cast<int>(item % groups) * SPW;
  struct alignas(EPL * sizeof(T)) Pack { T e[EPL]; };
  struct alignas(EPL * sizeof(W)) WPack { W e[EPL]; };
  struct alignas(EPL * 8) CsPack { float2 e[EPL]; };      // (cos, sin) of EPL consecutive pairs
  T* row = qkv + static_cast<size_t>(t) * row_stride + lane * EPL;
  Pack in[SPW];
#pragma unroll
  for (int i = 0; i < SPW; ++i)
    if (slot0 + i < slots) in[i] = *reinterpret_cast<const Pack*>(row + static_cast<size_t>(slot0 + i) * D);
  // what the row's slots share
  const bool any_kv = slot0 + SPW > heads;
  int m = -1;
  size_t cache_k = 0;                                      // offset of kv head 0's K row of this token in its page
  if (any_kv) {
    m = slot_mapping[t];
    if (m < 0 || m >= num_pages * page_size) {
      if (lane == 0 && m != kPaddingSlot) publish_error(error, kRowWithoutPage);   // (a row of padding is left alone)
      m = -1;
    } else {
      const int page = m / page_size, off = m % page_size;
      cache_k = static_cast<size_t>(page) * 2 * kv_heads * page_size * D + static_cast<size_t>(off) * D + lane * EPL;
    }
  }
  const size_t head_stride = static_cast<size_t>(page_size) * D;
  CsPack cs;
  if (rope != nullptr && slot0 < heads + kv_heads) {
    int pos = positions[t];
    if (pos < 0 || pos >= max_pos) {
      if (lane == 0) publish_error(error, kBadPosition);
      pos = 0;
    }
    cs = *reinterpret_cast<const CsPack*>(rope + (static_cast<size_t>(pos) * HALF + (lane & 15) * EPL) * 2);
  }
  WPack wq, wk;
  if (q_w != nullptr && slot0 < heads) wq = *reinterpret_cast<const WPack*>(q_w + lane * EPL);
  if (k_w != nullptr && slot0 + SPW > heads && slot0 < heads + kv_heads)
    wk = *reinterpret_cast<const WPack*>(k_w + lane * EPL);
#pragma unroll
  for (int i = 0; i < SPW; ++i) {
    const int slot = slot0 + i;
    if (slot >= slots) break;
    const bool is_q = slot < heads;
    const bool is_k = !is_q && slot < heads + kv_heads;
    T* dst_cache = nullptr;
    if (!is_q && m >= 0) dst_cache = cache + cache_k + static_cast<size_t>(slot - heads) * head_stride;   // K heads, then V heads
    if (!is_q && !is_k) {
      if (dst_cache != nullptr) *reinterpret_cast<Pack*>(dst_cache) = in[i];
      continue;
    }
    const bool normed = is_q ? q_w != nullptr : k_w != nullptr;
    float v[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) v[j] = to_float<T>(in[i].e[j]);
    head_norm_rotate<T, W, EPL>(v, normed ? (is_q ? wq.e : wk.e) : nullptr, eps, rope != nullptr ? cs.e : nullptr, lane);
    Pack outp;
#pragma unroll
    for (int j = 0; j < EPL; ++j) outp.e[j] = from_float<T>(v[j]);
    *reinterpret_cast<Pack*>(row + static_cast<size_t>(slot) * D) = outp;
    if (dst_cache != nullptr) *reinterpret_cast<Pack*>(dst_cache) = outp;
  }
}

// The same for many rows, with a head on 16 lanes (head_dim = 16 * EPL, EPL in {4, 8, 16}).  A lane holds EPL / 2
// elements of the head's first half and the EPL / 2 elements that rotate with them from the second half, so
// the rotation needs no exchange between lanes; the only shuffles are the four of the sum of squares (a shuffle
// costs the issue slots of four arithmetic instructions).  A warp works on two head slots at a time, SPW times.
// A group of slots that holds only V heads is copied to the cache and nothing else; a group of one kind (only q
// or only k heads: the usual case) reads one set of norm weights and selects nothing per element.
template <typename T, int N>
struct alignas(N * sizeof(T) > 16 ? 16 : N * sizeof(T)) VecPack {
  T e[N];
};

template <typename T, typename W, int EPL, int SPW, bool MIXED>
__device__ __forceinline__ void qk_wide_slots(const VecPack<T, EPL / 2> (&lo)[SPW], const VecPack<T, EPL / 2> (&hi)[SPW],
                                              T* __restrict__ row, T* __restrict__ cache, size_t cache_k,
                                              size_t head_stride, int m, int slot0, int sub, int slots, int heads,
                                              int kv_heads, const W* __restrict__ q_w, const W* __restrict__ k_w,
                                              int l16, float eps, const VecPack<float2, EPL / 2>& cs, bool has_rope) {
  constexpr int D = 16 * EPL, HALF = D / 2, E2 = EPL / 2;
  // wa: the weights of the group's first kind; wb (mixed groups only): the k weights behind q slots
  const bool first_is_q = slot0 < heads;
  const W* wa_src = first_is_q ? q_w : k_w;
  float wa_lo[E2], wa_hi[E2], wb_lo[E2], wb_hi[E2];
#pragma unroll
  for (int j = 0; j < E2; ++j) wa_lo[j] = wa_hi[j] = wb_lo[j] = wb_hi[j] = 1.0f;
  if (wa_src != nullptr) {
    const VecPack<W, E2> l = *reinterpret_cast<const VecPack<W, E2>*>(wa_src + l16 * E2);
    const VecPack<W, E2> h = *reinterpret_cast<const VecPack<W, E2>*>(wa_src + HALF + l16 * E2);
#pragma unroll
    for (int j = 0; j < E2; ++j) {
      wa_lo[j] = to_float<W>(l.e[j]);
      wa_hi[j] = to_float<W>(h.e[j]);
    }
  }
  if (MIXED && first_is_q && k_w != nullptr) {
    const VecPack<W, E2> l = *reinterpret_cast<const VecPack<W, E2>*>(k_w + l16 * E2);
    const VecPack<W, E2> h = *reinterpret_cast<const VecPack<W, E2>*>(k_w + HALF + l16 * E2);
#pragma unroll
    for (int j = 0; j < E2; ++j) {
      wb_lo[j] = to_float<W>(l.e[j]);
      wb_hi[j] = to_float<W>(h.e[j]);
    }
  }
#pragma unroll
  for (int i = 0; i < SPW; ++i) {
    const int slot = slot0 + 2 * i + sub;
    const bool live = slot < slots;
    const bool is_q = MIXED ? slot < heads : first_is_q;
    const bool is_k = MIXED ? (!is_q && slot < heads + kv_heads) : !first_is_q;
    const bool second = MIXED && first_is_q && !is_q;      // a k slot of a group that began with q slots
    const bool normed = is_q ? q_w != nullptr : (is_k && k_w != nullptr);
    float x[E2], y[E2];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < E2; ++j) {
      x[j] = to_float<T>(lo[i].e[j]);
      y[j] = to_float<T>(hi[i].e[j]);
      ss += x[j] * x[j];
      ss += y[j] * y[j];
    }
#pragma unroll
    for (int d = 8; d > 0; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);      // over the head's 16 lanes
    if (normed) {
      const float scale = 1.0f / sqrtf(ss / static_cast<float>(D) + eps);
#pragma unroll
      for (int j = 0; j < E2; ++j) {
        x[j] = round_to<T>((x[j] * scale) * (second ? wb_lo[j] : wa_lo[j]));
        y[j] = round_to<T>((y[j] * scale) * (second ? wb_hi[j] : wa_hi[j]));
      }
    }
    VecPack<T, E2> out_lo, out_hi;
#pragma unroll
    for (int j = 0; j < E2; ++j) {
      float a = x[j], b = y[j];
      if (has_rope) {
        a = __fsub_rn(__fmul_rn(x[j], cs.e[j].x), __fmul_rn(y[j], cs.e[j].y));
        b = __fadd_rn(__fmul_rn(y[j], cs.e[j].x), __fmul_rn(x[j], cs.e[j].y));
      }
      out_lo.e[j] = from_float<T>(a);
      out_hi.e[j] = from_float<T>(b);
    }
    if (!live) continue;
    T* dst_cache = (!is_q && m >= 0) ? cache + cache_k + static_cast<size_t>(slot - heads) * head_stride : nullptr;
    if (MIXED && !is_q && !is_k) {                         // a V head: copied as it is
      if (dst_cache != nullptr) {
        *reinterpret_cast<VecPack<T, E2>*>(dst_cache) = lo[i];
        *reinterpret_cast<VecPack<T, E2>*>(dst_cache + HALF) = hi[i];
      }
      continue;
    }
    // a k head whose place is the cache goes there only: nothing reads it from the row afterwards (a ninth of
    // the kernel's bytes with 16 + 8 + 8 heads)
    if (is_q || dst_cache == nullptr) {
      T* dst = row + static_cast<size_t>(slot) * D;
      *reinterpret_cast<VecPack<T, E2>*>(dst) = out_lo;
      *reinterpret_cast<VecPack<T, E2>*>(dst + HALF) = out_hi;
    }
    if (dst_cache != nullptr) {
      *reinterpret_cast<VecPack<T, E2>*>(dst_cache) = out_lo;
      *reinterpret_cast<VecPack<T, E2>*>(dst_cache + HALF) = out_hi;
    }
  }
}

// Blocks of four warps, at most 64 registers a thread for heads of up to 128: the kernel waits on memory, and
// what helps it is many resident warps (measured at 2048 rows of 16 + 8 + 8 heads of 128: 13.8 us against 15.2
// to 17 with eight slots per warp in blocks of eight warps; 256 rows: 3.7 against 4.6).
constexpr int QK_WIDE_SPW = 2, QK_WIDE_WARPS = 4;
template <typename T, typename W, int EPL, int SPW>
__global__ void __launch_bounds__(QK_WIDE_WARPS * 32, (EPL <= 8 && sizeof(T) == 2) ? 8 : 4)
qk_norm_rope_kv_wide_kernel(T* __restrict__ qkv, int row_stride, int rows, int heads, int kv_heads,
                            const W* __restrict__ q_w, const W* __restrict__ k_w, float eps,
                            const float* __restrict__ rope, int max_pos, const int* __restrict__ positions,
                            const int* __restrict__ slot_mapping, T* __restrict__ cache, int page_size,
                            int num_pages, int write_kv, uint32_t* error) {
  wait_for_prior_kernels();
  launch_dependents();                                   // (the next kernel's blocks may become resident and wait)
  constexpr int D = 16 * EPL, HALF = D / 2, E2 = EPL / 2;
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane >> 4, l16 = lane & 15;
  const int slots = heads + (write_kv ? 2 * kv_heads : 0);
  const int groups = (slots + 2 * SPW - 1) / (2 * SPW);
  const long long item = static_cast<long long>(blockIdx.x) * warps_per_block + warp;
  if (item >= static_cast<long long>(rows) * groups) return;
  const int t = static_cast<int>(item / groups);
  const int slot0 = static_cast<int>(item % groups) * 2 * SPW;
  const int slot_end = min(slot0 + 2 * SPW, slots);        // past the group's last live slot
  T* row = qkv + static_cast<size_t>(t) * row_stride + l16 * E2;
  // what the row's rotation angles and cache slot depend on is asked for first: the angles' load waits for the
  // position, and that wait then runs under the loads of the row itself
  int pos_raw = 0, m_raw = -1;
  if (rope != nullptr && slot0 < heads + kv_heads) pos_raw = positions[t];
  if (slot_end > heads) m_raw = slot_mapping[t];
  VecPack<T, E2> lo[SPW], hi[SPW];
#pragma unroll
  for (int i = 0; i < SPW; ++i) {
    const int slot = min(slot0 + 2 * i + sub, slots - 1);
    lo[i] = *reinterpret_cast<const VecPack<T, E2>*>(row + static_cast<size_t>(slot) * D);
    hi[i] = *reinterpret_cast<const VecPack<T, E2>*>(row + static_cast<size_t>(slot) * D + HALF);
  }
  int m = -1;
  size_t cache_k = 0;
  if (slot_end > heads) {
    m = m_raw;
    if (m < 0 || m >= num_pages * page_size) {
      if (lane == 0 && m != kPaddingSlot) publish_error(error, kRowWithoutPage);   // (a row of padding is left alone)
      m = -1;
    } else {
      const int page = m / page_size, off = m % page_size;
      cache_k = static_cast<size_t>(page) * 2 * kv_heads * page_size * D + static_cast<size_t>(off) * D + l16 * E2;
    }
  }
  const size_t head_stride = static_cast<size_t>(page_size) * D;
  if (slot0 >= heads + kv_heads) {                         // only V heads: a copy
    if (m < 0) return;
#pragma unroll
    for (int i = 0; i < SPW; ++i) {
      const int slot = slot0 + 2 * i + sub;
      if (slot >= slots) continue;
      T* dst = cache + cache_k + static_cast<size_t>(slot - heads) * head_stride;
      *reinterpret_cast<VecPack<T, E2>*>(dst) = lo[i];
      *reinterpret_cast<VecPack<T, E2>*>(dst + HALF) = hi[i];
    }
    return;
  }
  VecPack<float2, E2> cs;
#pragma unroll
  for (int j = 0; j < E2; ++j) cs.e[j] = make_float2(1.0f, 0.0f);
  if (rope != nullptr) {
    int pos = pos_raw;
    if (pos < 0 || pos >= max_pos) {
      if (lane == 0) publish_error(error, kBadPosition);
      pos = 0;
    }
    cs = *reinterpret_cast<const VecPack<float2, E2>*>(rope + (static_cast<size_t>(pos) * HALF + l16 * E2) * 2);
  }
  const bool one_kind = slot_end <= heads || (slot0 >= heads && slot_end <= heads + kv_heads);
  if (one_kind)
    qk_wide_slots<T, W, EPL, SPW, false>(lo, hi, row, cache, cache_k, head_stride, m, slot0, sub, slots, heads,
                                         kv_heads, q_w, k_w, l16, eps, cs, rope != nullptr);
  else
    qk_wide_slots<T, W, EPL, SPW, true>(lo, hi, row, cache, cache_k, head_stride, m, slot0, sub, slots, heads,
                                        kv_heads, q_w, k_w, l16, eps, cs, rope != nullptr);
}

// ---------------------------------------------------------------------------
// SiLU-mul: out[t,i] = round( (g / (1 + exp(-g))) * u ), g = in[t,i], u = in[t,I+i]
// (qwen_bf16_primitives.cu:274-283)
// ---------------------------------------------------------------------------
// Columns of gate_up come in blocks of 2 * il: il gate columns, then their il up columns (il = inter:
// all gates, then all ups).
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, long long rows,
                                int inter, int il) {
  wait_for_prior_kernels();
  launch_dependents();                                   // (the next kernel's blocks may become resident and wait)
  const long long total = rows * inter;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / inter;
    const int c = static_cast<int>(i - t * inter);
    const int gc = (c / il) * 2 * il + c % il;
    const float g = to_float<T>(gate_up[t * 2 * inter + gc]);
    const float u = to_float<T>(gate_up[t * 2 * inter + gc + il]);
    out[i] = from_float<T>((g / (1.0f + expf(-g))) * u);
  }
}

// gather rows of a matrix: out[i,:] = in[rows[i],:]
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ in, const int* __restrict__ rows,
                                   T* __restrict__ out, int width) {
  wait_for_prior_kernels();
  launch_dependents();                                   // (the next kernel's blocks may become resident and wait)
  const T* s = in + static_cast<size_t>(rows[blockIdx.x]) * width;
  T* d = out + static_cast<size_t>(blockIdx.x) * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) d[c] = s[c];
}

}  // namespace pih

using namespace pih;

int pih::g_dependent_launch = 1;

// 1 (the default): kernels of the pack are launched so that each may begin while the one before it drains
// (see common.cuh); 0: plain launches.  Returns the previous setting.
extern "C" int pih_set_dependent_launch(int on) {
  const int before = pih::g_dependent_launch;
  pih::g_dependent_launch = on ? 1 : 0;
  return before;
}

extern "C" int pih_embedding(int dtype, const void* table, const int* ids, void* out, int rows,
                             int hidden, int vocab, uint32_t* error, void* stream) {
  if (rows <= 0) return 0;
  if (hidden <= 0 || vocab <= 0) return PIH_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int threads = 128;
  if (dtype == PIH_F32)
    launch_kernel(embedding_kernel<float>, dim3(rows), dim3(threads), 0, s, static_cast<const float*>(table), ids,
                                                     static_cast<float*>(out), rows, hidden, vocab, error);
  else if (dtype == PIH_BF16)
    launch_kernel(embedding_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, s, 
        static_cast<const __nv_bfloat16*>(table), ids, static_cast<__nv_bfloat16*>(out), rows, hidden,
        vocab, error);
  else
    return PIH_ERR_BAD_ARGUMENT;
  PIH_LAUNCH_CHECK();
  return 0;
}

// Vectorised variant: 16-byte loads, the row kept in registers between the two passes.
// Needs width * sizeof(T) % 16 == 0 and width <= threads * VEC * CHUNKS.
template <typename T, typename W, int CHUNKS>
__global__ void rmsnorm_vec_kernel(T* __restrict__ x, const T* __restrict__ delta,
                                   const W* __restrict__ weight, T* __restrict__ out,
                                   const int* __restrict__ rows, int width, float eps) {
  wait_for_prior_kernels();
  launch_dependents();                                   // (the next kernel's blocks may become resident and wait)
  constexpr int VEC = 16 / sizeof(T);
  __shared__ float scratch[33];
  const int o = blockIdx.x;
  const size_t r = rows != nullptr ? static_cast<size_t>(rows[o]) : static_cast<size_t>(o);
  T* xr = x + r * width;
  const T* dr = delta != nullptr ? delta + r * width : nullptr;
  const bool write_back = delta != nullptr && rows == nullptr;
  const int nvec = width / VEC;
  float v[CHUNKS][VEC];
  float ss = 0.0f;
#pragma unroll
  for (int k = 0; k < CHUNKS; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < nvec) {
      uint4 raw = reinterpret_cast<const uint4*>(xr)[i];
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < VEC; ++j) v[k][j] = to_float<T>(e[j]);
      if (dr != nullptr) {
        uint4 draw = reinterpret_cast<const uint4*>(dr)[i];
        const T* d = reinterpret_cast<const T*>(&draw);
        uint4 packed;
        T* pk = reinterpret_cast<T*>(&packed);
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          pk[j] = from_float<T>(v[k][j] + to_float<T>(d[j]));
          v[k][j] = to_float<T>(pk[j]);
        }
        if (write_back) reinterpret_cast<uint4*>(xr)[i] = packed;
      }
#pragma unroll
      for (int j = 0; j < VEC; ++j) ss += v[k][j] * v[k][j];
    }
  }
  // (the weights are asked for before the block-wide sum: after it they would be one more trip to the cache on the
  // path of every row)
  float wv[CHUNKS][VEC];
#pragma unroll
  for (int k = 0; k < CHUNKS; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
#pragma unroll
    for (int j = 0; j < VEC; ++j) wv[k][j] = i < nvec ? to_float<W>(weight[i * VEC + j]) : 0.0f;
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / static_cast<float>(width) + eps);
  T* yr = out + static_cast<size_t>(o) * width;
#pragma unroll
  for (int k = 0; k < CHUNKS; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < nvec) {
      uint4 packed;
      T* pk = reinterpret_cast<T*>(&packed);
#pragma unroll
      for (int j = 0; j < VEC; ++j) pk[j] = from_float<T>((v[k][j] * scale) * wv[k][j]);
      reinterpret_cast<uint4*>(yr)[i] = packed;
    }
  }
}

// A warp per row, for steps of many rows: a lane holds CHUNKS 16-byte pieces of the row (piece lane + 32 k), all
// of their loads in flight at once, and the row's sum of squares needs shuffles only.  One block per row with a
// block-wide sum (above) has two 16-byte loads a thread in flight and two barriers on every row's path: on 2048
// rows of 1024 it ran at 2.7 TB/s out of the L2.  Needs width * sizeof(T) == 32 * CHUNKS * 16 and weights
// aligned to 16 bytes.
constexpr int NORM_ROWS_WARPS = 8;
template <typename T, typename W, int CHUNKS>
__global__ void __launch_bounds__(NORM_ROWS_WARPS * 32)
rmsnorm_rows_kernel(T* __restrict__ x, const T* __restrict__ delta, const W* __restrict__ weight,
                    T* __restrict__ out, const int* __restrict__ rows, int out_rows, int width, float eps) {
  wait_for_prior_kernels();
  launch_dependents();                                   // (the next kernel's blocks may become resident and wait)
  constexpr int VEC = 16 / sizeof(T);
  constexpr int WV = VEC * sizeof(W) / 16;               // 16-byte loads per VEC weights
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int o = blockIdx.x * NORM_ROWS_WARPS + warp;
  if (o >= out_rows) return;
  const size_t r = rows != nullptr ? static_cast<size_t>(rows[o]) : static_cast<size_t>(o);
  uint4* xr = reinterpret_cast<uint4*>(x + r * width);
  const uint4* dr = delta != nullptr ? reinterpret_cast<const uint4*>(delta + r * width) : nullptr;
  const bool write_back = delta != nullptr && rows == nullptr;
  uint4 h[CHUNKS], d[CHUNKS], wq[CHUNKS][WV];
#pragma unroll
  for (int k = 0; k < CHUNKS; ++k) h[k] = xr[lane + 32 * k];
  if (dr != nullptr) {
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) d[k] = dr[lane + 32 * k];
  }
  // (the weights too: asked for after the sum they would be one more trip to the cache on every row's path)
#pragma unroll
  for (int k = 0; k < CHUNKS; ++k)
#pragma unroll
    for (int u = 0; u < WV; ++u) wq[k][u] = reinterpret_cast<const uint4*>(weight)[(lane + 32 * k) * WV + u];
  float ss = 0.0f;
#pragma unroll
  for (int k = 0; k < CHUNKS; ++k) {
    T* e = reinterpret_cast<T*>(&h[k]);
    if (dr != nullptr) {
      const T* de = reinterpret_cast<const T*>(&d[k]);
#pragma unroll
      for (int j = 0; j < VEC; ++j) e[j] = from_float<T>(to_float<T>(e[j]) + to_float<T>(de[j]));
      if (write_back) xr[lane + 32 * k] = h[k];
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const float f = to_float<T>(e[j]);
      ss = fmaf(f, f, ss);
    }
  }
  ss = warp_sum(ss);
  const float scale = 1.0f / sqrtf(ss / static_cast<float>(width) + eps);
  uint4* yr = reinterpret_cast<uint4*>(out + static_cast<size_t>(o) * width);
#pragma unroll
  for (int k = 0; k < CHUNKS; ++k) {
    const W* we = reinterpret_cast<const W*>(wq[k]);
    T* e = reinterpret_cast<T*>(&h[k]);
#pragma unroll
    for (int j = 0; j < VEC; ++j) e[j] = from_float<T>((to_float<T>(e[j]) * scale) * to_float<W>(we[j]));
    yr[lane + 32 * k] = h[k];
  }
}

template <typename T, typename W>
static int launch_rmsnorm(void* x, const void* delta, const void* weight, void* out, const int* rows,
                          int out_rows, int width, float eps, cudaStream_t s) {
  constexpr int VEC = 16 / sizeof(T);
  // many rows, enough to give every SM a block of warps: a warp each (32 rows of 2048: 3.9 us against 3.0 with a
  // block per row, which then has the more loads in flight)
  if (out_rows >= 1024 && width % (32 * VEC) == 0 && width / (32 * VEC) <= 8 &&
      (reinterpret_cast<uintptr_t>(weight) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(delta) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    const int chunks = width / (32 * VEC);
    const dim3 grid((out_rows + NORM_ROWS_WARPS - 1) / NORM_ROWS_WARPS), block(NORM_ROWS_WARPS * 32);
    T* xp = static_cast<T*>(x);
    const T* dp = static_cast<const T*>(delta);
    const W* wp = static_cast<const W*>(weight);
    T* op = static_cast<T*>(out);
    bool taken = true;
    switch (chunks) {
      case 1: launch_kernel(rmsnorm_rows_kernel<T, W, 1>, grid, block, 0, s, xp, dp, wp, op, rows, out_rows, width, eps); break;
      case 2: launch_kernel(rmsnorm_rows_kernel<T, W, 2>, grid, block, 0, s, xp, dp, wp, op, rows, out_rows, width, eps); break;
      case 4: launch_kernel(rmsnorm_rows_kernel<T, W, 4>, grid, block, 0, s, xp, dp, wp, op, rows, out_rows, width, eps); break;
      case 8: launch_kernel(rmsnorm_rows_kernel<T, W, 8>, grid, block, 0, s, xp, dp, wp, op, rows, out_rows, width, eps); break;
      default: taken = false;
    }
    if (taken) {
      PIH_LAUNCH_CHECK();
      return 0;
    }
  }
  if ((width * sizeof(T)) % 16 == 0) {
    const int nvec = width / VEC;
    int threads = 32;
    while (threads < 256 && threads * 2 <= nvec) threads *= 2;         // 32..256
    if (nvec <= threads * 4) {
      T* xp = static_cast<T*>(x);
      const T* dp = static_cast<const T*>(delta);
      const W* wp = static_cast<const W*>(weight);
      T* op = static_cast<T*>(out);
      if (nvec <= threads)
        launch_kernel(rmsnorm_vec_kernel<T, W, 1>, dim3(out_rows), dim3(threads), 0, s, xp, dp, wp, op, rows, width, eps);
      else if (nvec <= threads * 2)
        launch_kernel(rmsnorm_vec_kernel<T, W, 2>, dim3(out_rows), dim3(threads), 0, s, xp, dp, wp, op, rows, width, eps);
      else
        launch_kernel(rmsnorm_vec_kernel<T, W, 4>, dim3(out_rows), dim3(threads), 0, s, xp, dp, wp, op, rows, width, eps);
      PIH_LAUNCH_CHECK();
      return 0;
    }
  }
  int threads = 256;
  if (width <= 128) threads = 32;
  else if (width <= 512) threads = 128;
  else if (width >= 4096) threads = 512;
  launch_kernel(rmsnorm_kernel<T, W>, dim3(out_rows), dim3(threads), 0, s, static_cast<T*>(x), static_cast<const T*>(delta),
                                                    static_cast<const W*>(weight), static_cast<T*>(out),
                                                    rows, width, eps);
  PIH_LAUNCH_CHECK();
  return 0;
}

// weight_dtype may be PIH_F32 with a bf16 stream (a norm weight stored in 32-bit stays so)
extern "C" int pih_rmsnorm(int dtype, int weight_dtype, void* x, const void* delta, const void* weight,
                           void* out, const int* rows, int out_rows, int width, float eps,
                           void* stream) {
  if (out_rows <= 0) return 0;
  if (width <= 0 || !(eps > 0.0f)) return PIH_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == PIH_F32 && weight_dtype == PIH_F32)
    return launch_rmsnorm<float, float>(x, delta, weight, out, rows, out_rows, width, eps, s);
  if (dtype == PIH_BF16 && weight_dtype == PIH_BF16)
    return launch_rmsnorm<__nv_bfloat16, __nv_bfloat16>(x, delta, weight, out, rows, out_rows, width, eps, s);
  if (dtype == PIH_BF16 && weight_dtype == PIH_F32)
    return launch_rmsnorm<__nv_bfloat16, float>(x, delta, weight, out, rows, out_rows, width, eps, s);
  return PIH_ERR_BAD_ARGUMENT;
}

template <typename T, typename W>
static int launch_qk(void* qkv, int row_stride, int rows, int heads, int kv_heads, int head_dim,
                     const void* q_w, const void* k_w, float eps, const float* rope, int rotary_dim,
                     int max_pos, const int* positions, const int* slot_mapping, void* cache,
                     int page_size, int num_pages, int write_kv, uint32_t* error, cudaStream_t s) {
  const long long items = static_cast<long long>(rows) * (heads + (write_kv ? 2 * kv_heads : 0));
  const bool whole_head = rope == nullptr || rotary_dim == head_dim;
  const auto aligned64 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 63) == 0; };
  if (whole_head && (head_dim == 64 || head_dim == 128 || head_dim == 256) &&
      (row_stride * sizeof(T)) % 16 == 0 && aligned64(qkv) && aligned64(q_w) && aligned64(k_w) && aligned64(rope) &&
      aligned64(cache)) {
    const int warps = 8;
    const int slots = heads + (write_kv ? 2 * kv_heads : 0);
    // with few rows (a decode step) one slot per warp is the shortest chain
    if (rows >= 64) {
      // many rows: a head on 16 lanes, four head slots per warp
      constexpr int SPW = QK_WIDE_SPW;
      const int warps = QK_WIDE_WARPS;
      const long long work = static_cast<long long>(rows) * ((slots + 2 * SPW - 1) / (2 * SPW));
      const unsigned blocks = static_cast<unsigned>((work + warps - 1) / warps);
#define PIH_QK_WIDE(EPL)                                                                                   \
  launch_kernel(qk_norm_rope_kv_wide_kernel<T, W, EPL, SPW>, dim3(blocks), dim3(warps * 32), 0, s,         \
      static_cast<T*>(qkv), row_stride, rows, heads, kv_heads, static_cast<const W*>(q_w),                 \
      static_cast<const W*>(k_w), eps, rope, max_pos, positions, slot_mapping, static_cast<T*>(cache),     \
      page_size, num_pages, write_kv, error)
      if (head_dim == 64) PIH_QK_WIDE(4);
      else if (head_dim == 128) PIH_QK_WIDE(8);
      else PIH_QK_WIDE(16);
#undef PIH_QK_WIDE
      PIH_LAUNCH_CHECK();
      return 0;
    }
    const int spw = 1;
    const long long work = static_cast<long long>(rows) * ((slots + spw - 1) / spw);
    const unsigned blocks = static_cast<unsigned>((work + warps - 1) / warps);
#define PIH_QK_FAST_SPW(EPL, SPW)                                                                          \
  launch_kernel(qk_norm_rope_kv_fast_kernel<T, W, EPL, SPW>, dim3(blocks), dim3(warps * 32), 0, s,         \
      static_cast<T*>(qkv), row_stride, rows, heads, kv_heads, static_cast<const W*>(q_w),                 \
      static_cast<const W*>(k_w), eps, rope, max_pos, positions, slot_mapping, static_cast<T*>(cache),     \
      page_size, num_pages, write_kv, error)
#define PIH_QK_FAST(EPL) PIH_QK_FAST_SPW(EPL, 1)
    if (head_dim == 64) PIH_QK_FAST(2);
    else if (head_dim == 128) PIH_QK_FAST(4);
    else PIH_QK_FAST(8);
#undef PIH_QK_FAST_SPW
#undef PIH_QK_FAST
    PIH_LAUNCH_CHECK();
    return 0;
  }
  const int warps = 4;
  const long long blocks = (items + warps - 1) / warps;
  const size_t smem = static_cast<size_t>(warps) * head_dim * sizeof(float);
  launch_kernel(qk_norm_rope_kv_kernel<T, W>, dim3(static_cast<unsigned>(blocks)), dim3(warps * 32), smem, s, 
      static_cast<T*>(qkv), row_stride, rows, heads, kv_heads, head_dim, static_cast<const W*>(q_w),
      static_cast<const W*>(k_w), eps, rope, rotary_dim, max_pos, positions, slot_mapping,
      static_cast<T*>(cache), page_size, num_pages, write_kv, error);
  PIH_LAUNCH_CHECK();
  return 0;
}

extern "C" int pih_qk_norm_rope_kv_write(int dtype, int weight_dtype, void* qkv, int row_stride, int rows,
                                         int heads, int kv_heads, int head_dim, const void* q_w,
                                         const void* k_w, float eps, const float* rope, int rotary_dim,
                                         int max_pos, const int* positions, const int* slot_mapping,
                                         void* cache, int page_size, int num_pages, int write_kv,
                                         uint32_t* error, void* stream) {
  if (rows <= 0) return 0;
  if (heads <= 0 || kv_heads <= 0 || head_dim <= 0 || head_dim > 1024 || rotary_dim < 0 ||
      rotary_dim > head_dim || (rotary_dim & 1) || page_size <= 0)
    return PIH_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == PIH_F32 && weight_dtype == PIH_F32)
    return launch_qk<float, float>(qkv, row_stride, rows, heads, kv_heads, head_dim, q_w, k_w, eps, rope,
                                   rotary_dim, max_pos, positions, slot_mapping, cache, page_size,
                                   num_pages, write_kv, error, s);
  if (dtype == PIH_BF16 && weight_dtype == PIH_BF16)
    return launch_qk<__nv_bfloat16, __nv_bfloat16>(qkv, row_stride, rows, heads, kv_heads, head_dim, q_w,
                                                   k_w, eps, rope, rotary_dim, max_pos, positions,
                                                   slot_mapping, cache, page_size, num_pages, write_kv,
                                                   error, s);
  if (dtype == PIH_BF16 && weight_dtype == PIH_F32)
    return launch_qk<__nv_bfloat16, float>(qkv, row_stride, rows, heads, kv_heads, head_dim, q_w, k_w, eps,
                                           rope, rotary_dim, max_pos, positions, slot_mapping, cache,
                                           page_size, num_pages, write_kv, error, s);
  return PIH_ERR_BAD_ARGUMENT;
}

// (silu_times: common.cuh.  The exact forms made this kernel instruction-bound on the bf16 stream: 11 us for
// 2048 x 3072 outputs against 7.7.)
// 16 bytes per thread and row, two rows per thread with their loads issued together; needs
// inter * sizeof(T) % 16 == 0 and il a multiple of the vector length.  grid (column vectors / 256, row pairs)
template <typename T>
__global__ void silu_mul_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, long long rows,
                                    int inter, int il) {
  wait_for_prior_kernels();
  launch_dependents();                                   // (the next kernel's blocks may become resident and wait)
  constexpr int VEC = 16 / sizeof(T);
  const int per_row = inter / VEC;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= per_row) return;
  const int col = c * VEC;
  const int gc = il == VEC ? 2 * col : (col / il) * 2 * il + col % il;
  for (long long t0 = 2LL * blockIdx.y; t0 < rows; t0 += 2LL * gridDim.y) {
    uint4 graw[2], uraw[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      if (t0 + r < rows) {
        graw[r] = *reinterpret_cast<const uint4*>(gate_up + (t0 + r) * 2 * inter + gc);
        uraw[r] = *reinterpret_cast<const uint4*>(gate_up + (t0 + r) * 2 * inter + gc + il);
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      if (t0 + r >= rows) break;
      const T* g = reinterpret_cast<const T*>(&graw[r]);
      const T* u = reinterpret_cast<const T*>(&uraw[r]);
      uint4 packed;
      T* pk = reinterpret_cast<T*>(&packed);
#pragma unroll
      for (int j = 0; j < VEC; ++j) pk[j] = from_float<T>(silu_times<T>(to_float<T>(g[j]), to_float<T>(u[j])));
      reinterpret_cast<uint4*>(out + (t0 + r) * inter)[c] = packed;
    }
  }
}

template <typename T>
static int launch_silu(const void* gate_up, void* out, long long rows, int inter, int il, cudaStream_t s) {
  const int threads = 256;
  if ((inter * sizeof(T)) % 16 == 0 && il % (16 / sizeof(T)) == 0) {
    const int per_row = inter / (16 / static_cast<int>(sizeof(T)));
    const long long pairs = (rows + 1) / 2;
    const dim3 grid((per_row + threads - 1) / threads, static_cast<unsigned>(pairs < 65535 ? pairs : 65535));
    launch_kernel(silu_mul_vec_kernel<T>, grid, dim3(threads), 0, s, static_cast<const T*>(gate_up), static_cast<T*>(out),
                  rows, inter, il);
  } else {
    const long long total = rows * inter;
    const unsigned blocks = static_cast<unsigned>(min((total + threads - 1) / threads, 148LL * 32));
    launch_kernel(silu_mul_kernel<T>, dim3(blocks), dim3(threads), 0, s, static_cast<const T*>(gate_up), static_cast<T*>(out), rows,
                                                  inter, il);
  }
  PIH_LAUNCH_CHECK();
  return 0;
}

// interleave: gate_up columns come in blocks of `interleave` gate columns followed by their up columns
// (interleave == inter: all gates, then all ups); it must divide inter.
extern "C" int pih_silu_mul(int dtype, const void* gate_up, void* out, long long rows, int inter,
                            int interleave, void* stream) {
  if (rows <= 0) return 0;
  if (inter <= 0 || interleave <= 0 || inter % interleave) return PIH_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == PIH_F32) return launch_silu<float>(gate_up, out, rows, inter, interleave, s);
  if (dtype == PIH_BF16) return launch_silu<__nv_bfloat16>(gate_up, out, rows, inter, interleave, s);
  return PIH_ERR_BAD_ARGUMENT;
}

extern "C" int pih_gather_rows(int dtype, const void* in, const int* rows, void* out, int out_rows,
                               int width, void* stream) {
  if (out_rows <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == PIH_F32)
    launch_kernel(gather_rows_kernel<float>, dim3(out_rows), dim3(128), 0, s, static_cast<const float*>(in), rows,
                                                       static_cast<float*>(out), width);
  else if (dtype == PIH_BF16)
    launch_kernel(gather_rows_kernel<__nv_bfloat16>, dim3(out_rows), dim3(128), 0, s, 
        static_cast<const __nv_bfloat16*>(in), rows, static_cast<__nv_bfloat16*>(out), width);
  else
    return PIH_ERR_BAD_ARGUMENT;
  PIH_LAUNCH_CHECK();
  return 0;
}
