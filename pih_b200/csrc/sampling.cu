// Sampling on the device: one block per row of logits.
//
// The reference samples with ONE THREAD per row and an in-place heapsort of
// the whole vocabulary (kernels/cuda/qwen_bf16_primitives.cu:894-999; CPU
// definition plugins/model-qwen3/qwen3_sampler.cpp:106-185).  The definition
// is kept: scaled = logit / temperature; suppressed ids are left out; order
// by scaled descending, ties to the lower id; greedy takes the first;
// otherwise keep the first top_k, weights exp(scaled - max), the shortest
// prefix whose share reaches top_p, then inverse CDF with
// u = (philox_word + 0.5) / 2^32.
//
// Instead of sorting, every "first place in sorted order where a running
// total reaches a threshold" is found by a 4 x 8-bit radix selection over
// the row: a prefix of the sorted order is the pair (key*, id*) — all
// elements with a larger key, and those with the same key and id <= id*.
// Masses are summed as 2^-44 fixed-point integers, so totals do not depend
// on the order of the atomic additions and a draw is reproducible bit for
// bit.  Totals differ from the reference's sequential float sums in the last
// places; a draw within that distance of a boundary may pick the neighbour.
#include "common.cuh"

namespace pih {

constexpr int kSampleThreads = 1024;
constexpr int kMaxSuppressed = 17;     // include/pih/model/qwen3_sampler.h:18
constexpr int kParamInts = 6 + kMaxSuppressed;
constexpr double kFixedOne = 17592186044416.0;   // 2^44

__device__ __forceinline__ uint32_t ordered_key(float x) {
  x += 0.0f;                                   // -0 -> +0: equal values, equal keys
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Philox4x32-10 keyed by the seed, counter (ordinal / 4, 0, 0), word ordinal % 4
// (plugins/model-qwen3/qwen3_sampler.cpp:85-104)
__device__ uint32_t philox_word(uint32_t key0, uint32_t key1, uint64_t ordinal) {
  const uint64_t block = ordinal >> 2;
  uint32_t c0 = static_cast<uint32_t>(block), c1 = static_cast<uint32_t>(block >> 32), c2 = 0, c3 = 0;
  for (int round = 0; round < 10; ++round) {
    const uint64_t p0 = static_cast<uint64_t>(0xD2511F53u) * c0;
    const uint64_t p1 = static_cast<uint64_t>(0xCD9E8D57u) * c2;
    const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c1 ^ key0;
    const uint32_t n1 = static_cast<uint32_t>(p1);
    const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c3 ^ key1;
    const uint32_t n3 = static_cast<uint32_t>(p0);
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    key0 += 0x9E3779B9u;
    key1 += 0xBB67AE85u;
  }
  const uint32_t w[4] = {c0, c1, c2, c3};
  return w[ordinal & 3];
}

struct RowView {
  const float* logits;
  int vocab;
  float inv_unused;
  float temperature;      // divisor (1 when greedy)
  float max_scaled;
  int nsup;
  const int* sup;         // in shared memory
};

__device__ __forceinline__ bool allowed(const RowView& rv, int id) {
  for (int s = 0; s < rv.nsup; ++s)
    if (rv.sup[s] == id) return false;
  return true;
}

__device__ __forceinline__ float scaled_of(const RowView& rv, int id) { return rv.logits[id] / rv.temperature; }

__device__ __forceinline__ unsigned long long mass_of(const RowView& rv, float scaled) {
  return __double2ull_rd(static_cast<double>(expf(scaled - rv.max_scaled)) * kFixedOne);
}

struct Prefix {
  uint32_t key;
  int id;
};

__device__ __forceinline__ bool member(const Prefix& p, uint32_t key, int id) {
  return key > p.key || (key == p.key && id <= p.id);
}

__device__ unsigned long long block_sum_u64(unsigned long long v, unsigned long long* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    unsigned long long t = lane < (blockDim.x >> 5) ? scratch[lane] : 0ull;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) t += __shfl_xor_sync(0xffffffffu, t, d);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// total count (use_mass = false) or mass of the members of `p`
__device__ unsigned long long prefix_total(const RowView& rv, const Prefix& p, bool use_mass,
                                           unsigned long long* scratch) {
  unsigned long long local = 0;
  for (int id = threadIdx.x; id < rv.vocab; id += blockDim.x) {
    if (!allowed(rv, id)) continue;
    const float s = scaled_of(rv, id);
    if (!member(p, ordered_key(s), id)) continue;
    local += use_mass ? mass_of(rv, s) : 1ull;
  }
  return block_sum_u64(local, scratch);
}

// First place, in sorted order among the members of `p`, where the running total
// (count or mass) reaches `target` (1 <= target <= total of p).
__device__ Prefix find_crossing(const RowView& rv, const Prefix& p, bool use_mass,
                                unsigned long long target, unsigned long long* hist /*256*/,
                                unsigned long long* scratch /*40*/, int* iscratch /*40*/) {
  __shared__ uint32_t s_prefix_val;
  __shared__ unsigned long long s_acc;
  if (threadIdx.x == 0) {
    s_prefix_val = 0;
    s_acc = 0;
  }
  uint32_t mask = 0;
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    const uint32_t want = s_prefix_val;
    // A warp adds up what its lanes have for the same digit and sends one atomic addition per digit: a row of
    // logits has most of its keys under two or three values of the leading digit (sign and exponent), and 150 000
    // additions to three words of shared memory, one after the other, took 2 ms a row.  (Integer sums: the
    // order does not matter.)
    for (int base = 0; base < rv.vocab; base += blockDim.x) {
      const int id = base + threadIdx.x;
      int digit = -1;
      unsigned long long a = 0ull;
      if (id < rv.vocab && allowed(rv, id)) {
        const float s = scaled_of(rv, id);
        const uint32_t key = ordered_key(s);
        if ((key & mask) == want && member(p, key, id)) {
          a = use_mass ? mass_of(rv, s) : 1ull;
          if (a) digit = static_cast<int>((key >> shift) & 255u);
        }
      }
      unsigned todo = __ballot_sync(0xffffffffu, digit >= 0);
      while (todo) {
        const int leader = __ffs(todo) - 1;
        const int d = __shfl_sync(0xffffffffu, digit, leader);
        const unsigned same = __ballot_sync(0xffffffffu, digit == d);
        unsigned long long v = digit == d ? a : 0ull;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if ((threadIdx.x & 31) == leader) atomicAdd(&hist[d], v);
        todo &= ~same;
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned long long acc = s_acc;
      int digit = 0;
      for (int d = 255; d >= 0; --d) {
        if (acc + hist[d] >= target) {
          digit = d;
          break;
        }
        acc += hist[d];
      }
      s_acc = acc;
      s_prefix_val = want | (static_cast<uint32_t>(digit) << shift);
    }
    mask |= 255u << shift;
    __syncthreads();
  }
  const uint32_t key_c = s_prefix_val;
  const unsigned long long acc = s_acc;
  // members with exactly this key share one weight; how many of them are needed
  const int chunk = (rv.vocab + blockDim.x - 1) / blockDim.x;
  const int lo = threadIdx.x * chunk, hi = min(rv.vocab, lo + chunk);
  int mine = 0;
  unsigned long long a0 = 1ull;
  for (int id = lo; id < hi; ++id) {
    if (!allowed(rv, id)) continue;
    const float s = scaled_of(rv, id);
    const uint32_t key = ordered_key(s);
    if (key == key_c && member(p, key, id)) {
      ++mine;
      if (use_mass) a0 = mass_of(rv, s);
    }
  }
  // exclusive scan of `mine` over the block, in thread order
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = mine;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += n;
  }
  __syncthreads();
  if (lane == 31) iscratch[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = lane < (blockDim.x >> 5) ? iscratch[lane] : 0;
    int wi = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, wi, d);
      if (lane >= d) wi += n;
    }
    iscratch[lane] = wi - w;          // exclusive prefix of the warp totals
    if (lane == 31) iscratch[32] = wi;  // number of ties
  }
  __syncthreads();
  const int before = iscratch[warp] + incl - mine;
  const int ties = iscratch[32];
  // every tie has weight a0 (> 0 where mass is used: a zero weight cannot reach the target)
  __shared__ unsigned long long s_a0;
  if (mine > 0 && before == 0) s_a0 = a0;
  __syncthreads();
  const unsigned long long w0 = use_mass ? s_a0 : 1ull;
  unsigned long long need = w0 ? (target - acc + w0 - 1) / w0 : 1ull;
  if (need < 1) need = 1;
  if (need > static_cast<unsigned long long>(ties)) need = ties;
  const int r = static_cast<int>(need);               // the r-th tie in id order, 1-based
  __shared__ int s_id;
  if (mine > 0 && before < r && r <= before + mine) {
    int seen = before;
    for (int id = lo; id < hi; ++id) {
      if (!allowed(rv, id)) continue;
      const uint32_t key = ordered_key(scaled_of(rv, id));
      if (key == key_c && member(p, key, id)) {
        if (++seen == r) {
          s_id = id;
          break;
        }
      }
    }
  }
  __syncthreads();
  Prefix out;
  out.key = key_c;
  out.id = s_id;
  __syncthreads();
  return out;
}

__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ fparams,
              const int* __restrict__ iparams, int* __restrict__ out_tokens, uint32_t* error) {
  wait_for_prior_kernels();
  launch_dependents();                                   // (the next kernel's blocks may become resident and wait)
  __shared__ int s_sup[kMaxSuppressed];
  __shared__ unsigned long long s_hist[256];
  __shared__ unsigned long long s_scratch[40];
  __shared__ int s_iscratch[40];
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  const int row = blockIdx.x;
  const float temperature = fparams[row * 2 + 0];
  const float top_p = fparams[row * 2 + 1];
  const int* ip = iparams + static_cast<size_t>(row) * kParamInts;
  const int top_k = ip[0];
  const int nsup = min(max(ip[5], 0), kMaxSuppressed);
  if (threadIdx.x < kMaxSuppressed) s_sup[threadIdx.x] = threadIdx.x < nsup ? ip[6 + threadIdx.x] : -1;
  __syncthreads();
  RowView rv;
  rv.logits = logits + static_cast<size_t>(row) * vocab;
  rv.vocab = vocab;
  rv.temperature = temperature > 0.0f ? temperature : 1.0f;
  rv.nsup = nsup;
  rv.sup = s_sup;
  rv.max_scaled = 0.0f;

  // maximum and its lowest id
  float best = -INFINITY;
  int best_id = 0x7fffffff;
  bool bad = false;
  for (int id = threadIdx.x; id < vocab; id += blockDim.x) {
    const float raw = rv.logits[id];
    if (!isfinite(raw)) bad = true;
    if (!allowed(rv, id)) continue;
    const float s = raw / rv.temperature;
    if (s > best || (s == best && id < best_id)) {
      best = s;
      best_id = id;
    }
  }
  if (bad) publish_error(error, kNonFiniteLogit);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, d);
    const int oi = __shfl_xor_sync(0xffffffffu, best_id, d);
    if (ov > best || (ov == best && oi < best_id)) {
      best = ov;
      best_id = oi;
    }
  }
  if (lane == 0) {
    s_val[warp] = best;
    s_idx[warp] = best_id;
  }
  __syncthreads();
  if (warp == 0) {
    best = lane < (blockDim.x >> 5) ? s_val[lane] : -INFINITY;
    best_id = lane < (blockDim.x >> 5) ? s_idx[lane] : 0x7fffffff;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, d);
      const int oi = __shfl_xor_sync(0xffffffffu, best_id, d);
      if (ov > best || (ov == best && oi < best_id)) {
        best = ov;
        best_id = oi;
      }
    }
    if (lane == 0) {
      s_val[0] = best;
      s_idx[0] = best_id;
    }
  }
  __syncthreads();
  best = s_val[0];
  best_id = s_idx[0];
  if (best_id == 0x7fffffff) best_id = 0;      // nothing finite and allowed: reported above
  if (!(temperature > 0.0f) || !isfinite(best)) {
    if (threadIdx.x == 0) out_tokens[row] = best_id;
    return;
  }
  rv.max_scaled = best;

  Prefix kept;
  kept.key = 0u;
  kept.id = 0x7fffffff;
  const int n_allowed = vocab - nsup;
  if (top_k > 0 && top_k < n_allowed)
    kept = find_crossing(rv, kept, false, static_cast<unsigned long long>(top_k), s_hist, s_scratch, s_iscratch);
  if (top_p < 1.0f) {
    const unsigned long long filtered = prefix_total(rv, kept, true, s_scratch);
    unsigned long long target = __double2ull_ru(static_cast<double>(top_p) * static_cast<double>(filtered));
    target = min(max(target, 1ull), filtered);
    kept = find_crossing(rv, kept, true, target, s_hist, s_scratch, s_iscratch);
  }
  const unsigned long long retained = prefix_total(rv, kept, true, s_scratch);
  const uint32_t word = philox_word(static_cast<uint32_t>(ip[1]), static_cast<uint32_t>(ip[2]),
                                    (static_cast<uint64_t>(static_cast<uint32_t>(ip[4])) << 32) |
                                        static_cast<uint32_t>(ip[3]));
  const double u = (static_cast<double>(word) + 0.5) / 4294967296.0;
  unsigned long long target = __double2ull_rd(u * static_cast<double>(retained)) + 1ull;
  target = min(max(target, 1ull), retained);
  const Prefix pick = find_crossing(rv, kept, true, target, s_hist, s_scratch, s_iscratch);
  if (threadIdx.x == 0) out_tokens[row] = pick.id;
}

// argmax per row, ties to the lower id (qwen_bf16_primitives.cu:761-807)
__global__ void __launch_bounds__(kSampleThreads)
argmax_kernel(const float* __restrict__ logits, int vocab, int* __restrict__ out_tokens, uint32_t* error) {
  wait_for_prior_kernels();
  launch_dependents();                                   // (the next kernel's blocks may become resident and wait)
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  const float* row = logits + static_cast<size_t>(blockIdx.x) * vocab;
  float best = -INFINITY;
  int best_id = 0x7fffffff;
  bool bad = false;
  for (int id = threadIdx.x; id < vocab; id += blockDim.x) {
    const float v = row[id];
    if (!isfinite(v)) bad = true;
    if (v > best || (v == best && id < best_id)) {
      best = v;
      best_id = id;
    }
  }
  if (bad) publish_error(error, kNonFiniteLogit);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, d);
    const int oi = __shfl_xor_sync(0xffffffffu, best_id, d);
    if (ov > best || (ov == best && oi < best_id)) {
      best = ov;
      best_id = oi;
    }
  }
  if (lane == 0) {
    s_val[warp] = best;
    s_idx[warp] = best_id;
  }
  __syncthreads();
  if (warp == 0) {
    best = lane < (blockDim.x >> 5) ? s_val[lane] : -INFINITY;
    best_id = lane < (blockDim.x >> 5) ? s_idx[lane] : 0x7fffffff;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, d);
      const int oi = __shfl_xor_sync(0xffffffffu, best_id, d);
      if (ov > best || (ov == best && oi < best_id)) {
        best = ov;
        best_id = oi;
      }
    }
    if (lane == 0) out_tokens[blockIdx.x] = best_id == 0x7fffffff ? 0 : best_id;
  }
}

// Two-stage argmax for long rows: stage 1 reduces a slice of the row per block to (value, id),
// stage 2 reduces the slices.  Ties go to the lower id in both stages.
__global__ void __launch_bounds__(256)
argmax_slices_kernel(const float* __restrict__ logits, int vocab, int slices, float* __restrict__ part_val,
                     int* __restrict__ part_idx, uint32_t* error) {
  wait_for_prior_kernels();
  launch_dependents();                                   // (the next kernel's blocks may become resident and wait)
  __shared__ float s_val[8];
  __shared__ int s_idx[8];
  const int row = blockIdx.y, slice = blockIdx.x;
  const float* base = logits + static_cast<size_t>(row) * vocab;
  const int per = (vocab + slices - 1) / slices;
  const int lo = slice * per, hi = min(vocab, lo + per);
  float best = -INFINITY;
  int best_id = 0x7fffffff;
  bool bad = false;
  for (int id = lo + threadIdx.x; id < hi; id += blockDim.x) {
    const float v = base[id];
    if (!isfinite(v)) bad = true;
    if (v > best || (v == best && id < best_id)) {
      best = v;
      best_id = id;
    }
  }
  if (bad) publish_error(error, kNonFiniteLogit);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, d);
    const int oi = __shfl_xor_sync(0xffffffffu, best_id, d);
    if (ov > best || (ov == best && oi < best_id)) {
      best = ov;
      best_id = oi;
    }
  }
  if (lane == 0) {
    s_val[warp] = best;
    s_idx[warp] = best_id;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (blockDim.x >> 5); ++w)
      if (s_val[w] > best || (s_val[w] == best && s_idx[w] < best_id)) {
        best = s_val[w];
        best_id = s_idx[w];
      }
    part_val[row * slices + slice] = best;
    part_idx[row * slices + slice] = best_id;
  }
}

__global__ void argmax_final_kernel(const float* __restrict__ part_val, const int* __restrict__ part_idx,
                                    int slices, int* __restrict__ out_tokens) {
  wait_for_prior_kernels();
  launch_dependents();                                   // (the next kernel's blocks may become resident and wait)
  const int row = blockIdx.x, lane = threadIdx.x;
  float best = -INFINITY;
  int best_id = 0x7fffffff;
  for (int s = lane; s < slices; s += 32) {
    const float v = part_val[row * slices + s];
    const int i = part_idx[row * slices + s];
    if (v > best || (v == best && i < best_id)) {
      best = v;
      best_id = i;
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, d);
    const int oi = __shfl_xor_sync(0xffffffffu, best_id, d);
    if (ov > best || (ov == best && oi < best_id)) {
      best = ov;
      best_id = oi;
    }
  }
  if (lane == 0) out_tokens[row] = best_id == 0x7fffffff ? 0 : best_id;
}

// The log-probability of the token that was chosen for a row: scaled[token] - logsumexp(scaled) over the ids that
// are not suppressed, scaled = logit / temperature (1 when greedy), as the reference returns it with every sampled
// token (plugins/model-qwen3/qwen3_sampler.cpp:116-126, :143).  One block a row, two passes over the row (maximum,
// then the sum of exponentials); every sum in 32-bit with an order that depends on the block size alone.  The
// reference adds the exponentials one after the other in float32, which over a vocabulary of 150 000 drops a few
// thousandths of the mass; this sum does not.
constexpr int kLogprobThreads = 256;
constexpr int kLogprobMaxSuppressed = 17;
__global__ void __launch_bounds__(kLogprobThreads)
selected_logprob_kernel(const float* __restrict__ logits, int vocab, const int* __restrict__ tokens,
                        const float* __restrict__ fparams, const int* __restrict__ iparams, int icolumns,
                        float* __restrict__ out, uint32_t* error) {
  wait_for_prior_kernels();
  launch_dependents();
  __shared__ float scratch[33];
  __shared__ int suppressed[kLogprobMaxSuppressed];
  const int row = blockIdx.x;
  const float* x = logits + static_cast<size_t>(row) * vocab;
  float temperature = fparams != nullptr ? fparams[row * 2] : 0.0f;
  if (!(temperature > 0.0f)) temperature = 1.0f;
  int nsup = 0;
  if (iparams != nullptr) {
    nsup = min(max(iparams[row * icolumns + 5], 0), kLogprobMaxSuppressed);
    if (threadIdx.x < nsup) suppressed[threadIdx.x] = iparams[row * icolumns + 6 + threadIdx.x];
  }
  __syncthreads();
  auto allowed = [&](int i) {
    for (int k = 0; k < nsup; ++k)
      if (suppressed[k] == i) return false;
    return true;
  };
  float m = -INFINITY;
  for (int i = threadIdx.x; i < vocab; i += kLogprobThreads)
    if (nsup == 0 || allowed(i)) m = fmaxf(m, x[i] / temperature);
  // block maximum
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < kLogprobThreads / 32 ? scratch[threadIdx.x] : -INFINITY;
    v = warp_max(v);
    if (threadIdx.x == 0) scratch[32] = v;
  }
  __syncthreads();
  m = scratch[32];
  float sum = 0.0f;
  for (int i = threadIdx.x; i < vocab; i += kLogprobThreads)
    if (nsup == 0 || allowed(i)) sum += expf(x[i] / temperature - m);
  sum = block_sum(sum, scratch);
  if (threadIdx.x == 0) {
    const int tok = tokens[row];
    float lp = -INFINITY;
    if (tok >= 0 && tok < vocab && sum > 0.0f) lp = x[tok] / temperature - (m + logf(sum));
    if (!isfinite(lp)) publish_error(error, kNonFiniteLogit);
    out[row] = lp;
  }
}

}  // namespace pih

using namespace pih;

// out[row] = log-probability of tokens[row] under the row's scaled logits.  fparams [rows, 2] (temperature, top_p)
// and iparams [rows, icolumns] (column 5: the number of suppressed ids, columns 6..: the ids) as pih_sample takes
// them, or both null: temperature 1, nothing suppressed (the greedy path).
extern "C" int pih_selected_logprob(const float* logits, int rows, int vocab, const int* tokens, const float* fparams,
                                    const int* iparams, int icolumns, float* out, uint32_t* error, void* stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || (iparams != nullptr && icolumns < 6 + kLogprobMaxSuppressed)) return PIH_ERR_BAD_ARGUMENT;
  launch_kernel(selected_logprob_kernel, dim3(rows), dim3(kLogprobThreads), 0, static_cast<cudaStream_t>(stream), logits,
                vocab, tokens, fparams, iparams, icolumns, out, error);
  PIH_LAUNCH_CHECK();
  return 0;
}

// scratch: rows * 64 floats followed by rows * 64 ints (used when vocab is large); may be null,
// in which case one block reduces each row.
extern "C" int pih_argmax(const float* logits, int rows, int vocab, int* out_tokens, void* scratch,
                          uint32_t* error, void* stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) return PIH_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (scratch != nullptr && vocab >= 8192 && rows <= 65535) {
    const int slices = 64;
    float* pv = static_cast<float*>(scratch);
    int* pi = reinterpret_cast<int*>(pv + static_cast<size_t>(rows) * slices);
    launch_kernel(argmax_slices_kernel, dim3(dim3(slices, rows)), dim3(256), 0, s, logits, vocab, slices, pv, pi, error);
    PIH_LAUNCH_CHECK();
    launch_kernel(argmax_final_kernel, dim3(rows), dim3(32), 0, s, pv, pi, slices, out_tokens);
    PIH_LAUNCH_CHECK();
    return 0;
  }
  launch_kernel(argmax_kernel, dim3(rows), dim3(kSampleThreads), 0, s, logits, vocab, out_tokens, error);
  PIH_LAUNCH_CHECK();
  return 0;
}

// fparams [rows, 2] = (temperature, top_p); iparams [rows, 23] =
// (top_k or 0, seed lo, seed hi, ordinal lo, ordinal hi, n suppressed, 17 suppressed ids)
extern "C" int pih_sample(const float* logits, int rows, int vocab, const float* fparams,
                          const int* iparams, int* out_tokens, uint32_t* error, void* stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) return PIH_ERR_BAD_ARGUMENT;
  launch_kernel(sample_kernel, dim3(rows), dim3(kSampleThreads), 0, static_cast<cudaStream_t>(stream), logits, vocab, fparams,
                                                                                  iparams, out_tokens, error);
  PIH_LAUNCH_CHECK();
  return 0;
}
