// Sampling on the device: a thread-block cluster per row of logits.
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

// ---- a row is sampled by a CLUSTER of blocks ---------------------------------------------------------------------
// One block a row (what this kernel was first) made a row's eight to twenty passes over 150 000 logits the work
// of one SM: 0.84 ms for a step's sampled rows however few, on top of a decode step of 1 ms.  Now block c of a
// cluster of kSampleCluster takes the ids [c V/C, (c+1) V/C) of the row.  Whatever the single block summed over the
// row — the maximum, masses, the 256 counts of a radix pass, the number of ties — each block sums over its part
// and the blocks exchange through distributed shared memory: a block writes its words into one of two exchange
// areas in turn, a cluster barrier follows, and every block reads all blocks' words and combines them in rank order,
// so all blocks go on with the same values.  (Two areas: a block can only be one barrier ahead of the slowest
// reader.)  Sums are integers, so nothing depends on how the row is cut.
constexpr int kSampleCluster = 8;
constexpr int kSampleBlock = 1024;                        // the most threads of a block (see pih_sample for the choice)
constexpr int kExchangeWords = 4;
constexpr int kSampleCopies = 8;

__device__ __forceinline__ uint32_t sample_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void sample_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ unsigned long long load_u64_from_block(const unsigned long long* local, uint32_t rank) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(local));
  uint32_t remote;
  unsigned long long v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(a), "r"(rank));
  asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(remote) : "memory");
  return v;
}

__device__ __forceinline__ uint32_t load_u32_from_block(const uint32_t* local, uint32_t rank) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(local));
  uint32_t remote, v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(a), "r"(rank));
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(remote) : "memory");
  return v;
}

struct SampleShared {
  // this block's counts of a radix pass, two in turn, as three limbs of 15 bits each summed in 32 bits (a block's
  // part is at most 2^16 ids): 32-bit additions to shared memory are one instruction, 64-bit ones a loop
  uint32_t hist[2][3][256];
  // Copies of the counts for pairs of warps: a row's masses fall on few digits, and additions to one word of shared
  // memory are done one after the other whichever warps they come from (measured: one copy a block 70 us a pass;
  // adding up a warp's lanes per digit first — match.any, redux.sync — no better, because a warp's dozen distinct
  // digits are worked off one after the other as well).
  uint32_t priv[kSampleCopies][3][256];
  unsigned long long ghist[256];                         // the row's
  unsigned long long mine[2][kExchangeWords];            // this block's words of an exchange, two in turn
  unsigned long long all[kSampleCluster][kExchangeWords];
  unsigned long long scratch[40];
  int iscratch[40];
  int sup[kMaxSuppressed];
  float val[32];
  int idx[32];
  uint32_t prefix_val;
  unsigned long long acc;
  unsigned long long a0;
  int found;
};

struct RowView {
  const float* logits;
  int vocab;
  int lo, hi;             // this block's ids
  const float* staged;    // scaled values of this block's ids in shared memory, or null (the part does not fit)
  float temperature;      // divisor (1 when greedy)
  float max_scaled;
  int nsup;
  const int* sup;         // in shared memory
  int phase;              // which exchange area / counts come next
  int hphase;
  uint32_t rank;
};

__device__ __forceinline__ bool allowed(const RowView& rv, int id) {
  for (int s = 0; s < rv.nsup; ++s)
    if (rv.sup[s] == id) return false;
  return true;
}

__device__ __forceinline__ float scaled_of(const RowView& rv, int id) {
  return rv.staged != nullptr ? rv.staged[id - rv.lo] : rv.logits[id] / rv.temperature;
}

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

// Every block gives kExchangeWords words (thread 0's `w`) and gets all blocks' words in sm.all[rank][word].
// Called by every thread of every block of the cluster.
__device__ void exchange(SampleShared& sm, RowView& rv, const unsigned long long (&w)[kExchangeWords]) {
  if (threadIdx.x == 0) {
#pragma unroll
    for (int k = 0; k < kExchangeWords; ++k) sm.mine[rv.phase][k] = w[k];
  }
  sample_cluster_sync();                               // (a block barrier too: thread 0's stores are in place)
  if (threadIdx.x < kSampleCluster * kExchangeWords)
    sm.all[threadIdx.x / kExchangeWords][threadIdx.x % kExchangeWords] =
        load_u64_from_block(&sm.mine[rv.phase][threadIdx.x % kExchangeWords], threadIdx.x / kExchangeWords);
  __syncthreads();
  rv.phase ^= 1;
}

// total count (use_mass = false) or mass of the members of `p`, over the whole row
__device__ unsigned long long prefix_total(SampleShared& sm, RowView& rv, const Prefix& p, bool use_mass) {
  unsigned long long local = 0;
  for (int id = rv.lo + threadIdx.x; id < rv.hi; id += blockDim.x) {
    if (!allowed(rv, id)) continue;
    const float s = scaled_of(rv, id);
    if (!member(p, ordered_key(s), id)) continue;
    local += use_mass ? mass_of(rv, s) : 1ull;
  }
  const unsigned long long w[kExchangeWords] = {block_sum_u64(local, sm.scratch), 0ull, 0ull, 0ull};
  exchange(sm, rv, w);
  unsigned long long total = 0;
#pragma unroll
  for (int r = 0; r < kSampleCluster; ++r) total += sm.all[r][0];
  __syncthreads();
  return total;
}

// First place, in sorted order among the members of `p`, where the running total (count or mass) reaches a target
// (1 <= target <= total of p).  The target is `target` itself (kTargetGiven), or follows from the total of p, which
// the first radix pass yields on the way (a pass over the row saved): the least total that is at least `share` of
// it (kTargetShare: top_p) or the place of the draw `share` in it (kTargetDraw).
enum TargetKind { kTargetGiven, kTargetShare, kTargetDraw };
__device__ Prefix find_crossing(SampleShared& sm, RowView& rv, const Prefix& p, bool use_mass, TargetKind kind,
                                unsigned long long target, double share) {
  if (threadIdx.x == 0) {
    sm.prefix_val = 0;
    sm.acc = 0;
  }
  uint32_t mask = 0;
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    uint32_t (*hist)[256] = sm.hist[rv.hphase];
    uint32_t (*mine)[256] = sm.priv[(threadIdx.x >> 5) % kSampleCopies];
    for (int i = threadIdx.x; i < kSampleCopies * 3 * 256; i += blockDim.x) (&sm.priv[0][0][0])[i] = 0;
    __syncthreads();
    const uint32_t want = sm.prefix_val;
    for (int id = rv.lo + threadIdx.x; id < rv.hi; id += blockDim.x) {
      if (!allowed(rv, id)) continue;
      const float s = scaled_of(rv, id);
      const uint32_t key = ordered_key(s);
      if ((key & mask) != want || !member(p, key, id)) continue;
      const unsigned long long a = use_mass ? mass_of(rv, s) : 1ull;
      if (a == 0ull) continue;
      const int digit = static_cast<int>((key >> shift) & 255u);
      // a mass is at most 2^44: three limbs of 15 bits
      const uint32_t a0 = static_cast<uint32_t>(a) & 0x7FFFu, a1 = static_cast<uint32_t>(a >> 15) & 0x7FFFu,
                     a2 = static_cast<uint32_t>(a >> 30);
      if (a0) atomicAdd(&mine[0][digit], a0);
      if (a1) atomicAdd(&mine[1][digit], a1);
      if (a2) atomicAdd(&mine[2][digit], a2);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 3 * 256; i += blockDim.x) {
      uint32_t t = 0;
#pragma unroll
      for (int c = 0; c < kSampleCopies; ++c) t += (&sm.priv[c][0][0])[i];
      (&hist[0][0])[i] = t;
    }
    sample_cluster_sync();                             // every block's counts are complete
    for (int i = threadIdx.x; i < 256; i += blockDim.x) {
      uint32_t part[kSampleCluster][3];
#pragma unroll
      for (int r = 0; r < kSampleCluster; ++r)                 // (all on their way at once)
#pragma unroll
        for (int k = 0; k < 3; ++k) part[r][k] = load_u32_from_block(&hist[k][i], r);
      unsigned long long g = 0;
#pragma unroll
      for (int r = 0; r < kSampleCluster; ++r)
        g += static_cast<unsigned long long>(part[r][0]) + (static_cast<unsigned long long>(part[r][1]) << 15) +
             (static_cast<unsigned long long>(part[r][2]) << 30);
      sm.ghist[i] = g;
    }
    rv.hphase ^= 1;
    __syncthreads();
    if (pass == 0 && kind != kTargetGiven) {
      // the total of p: the sum of the first pass's counts (every block has the same counts and finds the same)
      unsigned long long total = 0;
      for (int i = 0; i < 256; ++i) total += sm.ghist[i];
      if (kind == kTargetShare) target = __double2ull_ru(share * static_cast<double>(total));
      else target = __double2ull_rd(share * static_cast<double>(total)) + 1ull;
      target = min(max(target, 1ull), total);
    }
    // the digit at which the running total, from the largest digit down, reaches the target: warp 0, a lane per
    // eight digits (lane 0 the largest), a scan over the lanes' sums, then the lane that holds the crossing walks
    // its eight
    if (threadIdx.x < 32) {
      const int ln = threadIdx.x;
      unsigned long long eight[8], sum = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        eight[j] = sm.ghist[255 - (ln * 8 + j)];
        sum += eight[j];
      }
      unsigned long long incl = sum;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const unsigned long long n = __shfl_up_sync(0xffffffffu, incl, d);
        if (ln >= d) incl += n;
      }
      const unsigned long long base = sm.acc + incl - sum;      // the total before this lane's digits
      const bool here = base < target && base + sum >= target;
      const unsigned found = __ballot_sync(0xffffffffu, here);
      // (a target beyond the row's total cannot happen: callers clamp it; digit 0 then)
      if (found == 0u ? ln == 31 : ln == __ffs(found) - 1) {
        unsigned long long acc = base;
        int digit = 0;
        if (found != 0u) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (acc + eight[j] >= target) {
              digit = 255 - (ln * 8 + j);
              break;
            }
            acc += eight[j];
          }
        } else {
          acc = base + sum;
        }
        sm.acc = acc;
        sm.prefix_val = want | (static_cast<uint32_t>(digit) << shift);
      }
    }
    mask |= 255u << shift;
    __syncthreads();
  }
  const uint32_t key_c = sm.prefix_val;
  const unsigned long long acc = sm.acc;
  // members with exactly this key share one weight; how many of them are needed.  Ties are counted in id order:
  // a thread takes a run of consecutive ids of this block's part, and the blocks' parts follow one another.
  const int span = rv.hi - rv.lo;
  const int chunk = (span + blockDim.x - 1) / blockDim.x;
  const int lo = rv.lo + threadIdx.x * chunk, hi = min(rv.hi, lo + chunk);
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
  if (lane == 31) sm.iscratch[warp] = incl;
  if (threadIdx.x == 0) sm.a0 = 0ull;
  __syncthreads();
  if (warp == 0) {
    int w = lane < (blockDim.x >> 5) ? sm.iscratch[lane] : 0;
    int wi = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, wi, d);
      if (lane >= d) wi += n;
    }
    sm.iscratch[lane] = wi - w;          // exclusive prefix of the warp totals
    if (lane == 31) sm.iscratch[32] = wi;  // this block's ties
  }
  __syncthreads();
  const int before_in_block = sm.iscratch[warp] + incl - mine;
  const int block_ties = sm.iscratch[32];
  if (mine > 0 && before_in_block == 0) sm.a0 = a0;       // (every tie has the same weight)
  __syncthreads();
  {
    const unsigned long long w[kExchangeWords] = {static_cast<unsigned long long>(block_ties), sm.a0, 0ull, 0ull};
    exchange(sm, rv, w);
  }
  int ties = 0, before_block = 0;
  unsigned long long w0 = 1ull;
  bool have = false;
#pragma unroll
  for (int r = 0; r < kSampleCluster; ++r) {
    const int t = static_cast<int>(sm.all[r][0]);
    if (static_cast<uint32_t>(r) < rv.rank) before_block += t;
    if (t > 0 && !have) {
      w0 = sm.all[r][1];
      have = true;
    }
    ties += t;
  }
  if (!use_mass) w0 = 1ull;
  // every tie has weight w0 (> 0 where mass is used: a zero weight cannot reach the target)
  unsigned long long need = w0 ? (target - acc + w0 - 1) / w0 : 1ull;
  if (need < 1) need = 1;
  if (need > static_cast<unsigned long long>(ties)) need = ties;
  const int r = static_cast<int>(need);               // the r-th tie in id order, 1-based
  const int before = before_block + before_in_block;
  if (threadIdx.x == 0) sm.found = -1;
  __syncthreads();
  if (mine > 0 && before < r && r <= before + mine) {
    int seen = before;
    for (int id = lo; id < hi; ++id) {
      if (!allowed(rv, id)) continue;
      const uint32_t key = ordered_key(scaled_of(rv, id));
      if (key == key_c && member(p, key, id)) {
        if (++seen == r) {
          sm.found = id;
          break;
        }
      }
    }
  }
  __syncthreads();
  {
    const unsigned long long w[kExchangeWords] = {static_cast<unsigned long long>(static_cast<long long>(sm.found)), 0ull, 0ull, 0ull};
    exchange(sm, rv, w);
  }
  Prefix out;
  out.key = key_c;
  out.id = 0;
#pragma unroll
  for (int q = 0; q < kSampleCluster; ++q) {
    const long long f = static_cast<long long>(sm.all[q][0]);
    if (f >= 0) out.id = static_cast<int>(f);
  }
  __syncthreads();
  return out;
}

__global__ void __launch_bounds__(kSampleBlock)
sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ fparams,
              const int* __restrict__ iparams, int* __restrict__ out_tokens, int staged_floats, uint32_t* error) {
  wait_for_prior_kernels();
  launch_dependents();                                   // (the next kernel's blocks may become resident and wait)
  __shared__ SampleShared sm;
  const int row = blockIdx.x / kSampleCluster;
  const float temperature = fparams[row * 2 + 0];
  const float top_p = fparams[row * 2 + 1];
  const int* ip = iparams + static_cast<size_t>(row) * kParamInts;
  const int top_k = ip[0];
  const int nsup = min(max(ip[5], 0), kMaxSuppressed);
  if (threadIdx.x < kMaxSuppressed) sm.sup[threadIdx.x] = threadIdx.x < nsup ? ip[6 + threadIdx.x] : -1;
  __syncthreads();
  RowView rv;
  rv.logits = logits + static_cast<size_t>(row) * vocab;
  rv.vocab = vocab;
  rv.rank = sample_cluster_rank();
  const int part = (vocab + kSampleCluster - 1) / kSampleCluster;
  rv.lo = min(vocab, static_cast<int>(rv.rank) * part);
  rv.hi = min(vocab, rv.lo + part);
  rv.temperature = temperature > 0.0f ? temperature : 1.0f;
  rv.nsup = nsup;
  rv.sup = sm.sup;
  rv.max_scaled = 0.0f;
  rv.phase = 0;
  rv.hphase = 0;
  rv.staged = nullptr;

  // The block's part of the row goes to shared memory once, divided by the temperature: the passes that follow read
  // it eight to twenty times.  From global memory a pass was bound by latency (a thread had one 4-byte load in
  // flight at a time, between the warp votes of the counting loop: 13 us a pass), and every pass paid the division
  // again.  These loads do not depend on one another and go out back to back.
  extern __shared__ float staged_part[];
  bool bad = false;
  // maximum and its lowest id, found on the way
  float best = -INFINITY;
  int best_id = 0x7fffffff;
  const bool stage = staged_floats >= rv.hi - rv.lo;
  for (int id = rv.lo + threadIdx.x; id < rv.hi; id += blockDim.x) {
    const float raw = rv.logits[id];
    if (!isfinite(raw)) bad = true;
    const float s = raw / rv.temperature;
    if (stage) staged_part[id - rv.lo] = s;
    if (!allowed(rv, id)) continue;
    if (s > best || (s == best && id < best_id)) {
      best = s;
      best_id = id;
    }
  }
  if (stage) rv.staged = staged_part;                    // (read only after the block barriers of the reduction below)
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
    sm.val[warp] = best;
    sm.idx[warp] = best_id;
  }
  __syncthreads();
  if (warp == 0) {
    best = lane < (blockDim.x >> 5) ? sm.val[lane] : -INFINITY;
    best_id = lane < (blockDim.x >> 5) ? sm.idx[lane] : 0x7fffffff;
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
      sm.val[0] = best;
      sm.idx[0] = best_id;
    }
  }
  __syncthreads();
  {
    const unsigned long long w[kExchangeWords] = {static_cast<unsigned long long>(__float_as_uint(sm.val[0])),
                                                  static_cast<unsigned long long>(static_cast<uint32_t>(sm.idx[0])), 0ull, 0ull};
    exchange(sm, rv, w);
  }
  best = -INFINITY;
  best_id = 0x7fffffff;
#pragma unroll
  for (int r = 0; r < kSampleCluster; ++r) {             // the blocks' ids ascend with their rank: the first maximum has the lowest id
    const float v = __uint_as_float(static_cast<uint32_t>(sm.all[r][0]));
    const int i = static_cast<int>(static_cast<uint32_t>(sm.all[r][1]));
    if (v > best || (v == best && i < best_id)) {
      best = v;
      best_id = i;
    }
  }
  __syncthreads();
  if (best_id == 0x7fffffff) best_id = 0;      // nothing finite and allowed: reported above
  if (!(temperature > 0.0f) || !isfinite(best)) {        // (every block of the cluster sees the same and leaves)
    if (threadIdx.x == 0 && rv.rank == 0) out_tokens[row] = best_id;
    sample_cluster_sync();                               // (another block may still be reading this one's words)
    return;
  }
  rv.max_scaled = best;

  Prefix kept;
  kept.key = 0u;
  kept.id = 0x7fffffff;
  const int n_allowed = vocab - nsup;
  if (top_k > 0 && top_k < n_allowed)
    kept = find_crossing(sm, rv, kept, false, kTargetGiven, static_cast<unsigned long long>(top_k), 0.0);
  if (top_p < 1.0f) {
    kept = find_crossing(sm, rv, kept, true, kTargetShare, 0ull, static_cast<double>(top_p));
  }
  const uint32_t word = philox_word(static_cast<uint32_t>(ip[1]), static_cast<uint32_t>(ip[2]),
                                    (static_cast<uint64_t>(static_cast<uint32_t>(ip[4])) << 32) |
                                        static_cast<uint32_t>(ip[3]));
  const double u = (static_cast<double>(word) + 0.5) / 4294967296.0;
  const Prefix pick = find_crossing(sm, rv, kept, true, kTargetDraw, 0ull, u);
  if (threadIdx.x == 0 && rv.rank == 0) out_tokens[row] = pick.id;
  sample_cluster_sync();                                 // nobody leaves while another block may still read its words
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


// ---------------------------------------------------------------------------------------------------------
// The most probable ids of a row with their log-probabilities under the row's scaled logits
// (plugins/model-qwen3/qwen3_sampler.cpp:118-143: logits / temperature, suppressed ids left out, ordered by
// value, then by id; at most 20 of them; the choice of top-k / top-p plays no part).  Two kernels: a block a
// (row, slice of the vocabulary) keeps its slice in shared memory and takes `count` maxima out of it one after
// the other, with the slice's maximum and its sum of exponentials; a block a row then merges the slices.
constexpr int kTopLogprobsMax = 20;
constexpr int kTopThreads = 512;
constexpr int kTopSliceFloats = 40 * 1024;      // 160 KB of shared memory at most
constexpr int kTopMaxSlices = 64;

// the better of two (value, id): the larger value, the smaller id among equals (-1: none)
__device__ __forceinline__ void keep_better(float& v, int& i, float ov, int oi) {
  if (oi >= 0 && (i < 0 || ov > v || (ov == v && oi < i))) {
    v = ov;
    i = oi;
  }
}
// the best (value, id) of the block, to every thread; scratch_v / scratch_i hold 33 words each
__device__ void block_best(float& v, int& i, float* scratch_v, int* scratch_i) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, d);
    const int oi = __shfl_xor_sync(0xffffffffu, i, d);
    keep_better(v, i, ov, oi);
  }
  __syncthreads();
  if (lane == 0) {
    scratch_v[warp] = v;
    scratch_i[warp] = i;
  }
  __syncthreads();
  if (warp == 0) {
    float bv = lane < warps ? scratch_v[lane] : 0.0f;
    int bi = lane < warps ? scratch_i[lane] : -1;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, d);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, d);
      keep_better(bv, bi, ov, oi);
    }
    if (lane == 0) {
      scratch_v[32] = bv;
      scratch_i[32] = bi;
    }
  }
  __syncthreads();
  v = scratch_v[32];
  i = scratch_i[32];
}

// part_v / part_i: [rows, slices, count] candidates; part_ms: [rows, slices, 2] (maximum, sum of exp(x - maximum))
__global__ void __launch_bounds__(kTopThreads)
top_logprobs_slices_kernel(const float* __restrict__ logits, int vocab, int count, int slice_len,
                           const float* __restrict__ fparams, const int* __restrict__ iparams, int icolumns,
                           float* __restrict__ part_v, int* __restrict__ part_i, float* __restrict__ part_ms,
                           uint32_t* error) {
  wait_for_prior_kernels();
  launch_dependents();
  extern __shared__ float slice[];
  __shared__ float scratch_v[33];
  __shared__ int scratch_i[33];
  __shared__ int suppressed[kLogprobMaxSuppressed];
  const int row = blockIdx.y, sl = blockIdx.x, slices = gridDim.x;
  const int lo = sl * slice_len, n = max(0, min(vocab - lo, slice_len));
  const float* x = logits + static_cast<size_t>(row) * vocab + lo;
  float temperature = fparams != nullptr ? fparams[row * 2] : 0.0f;
  if (!(temperature > 0.0f)) temperature = 1.0f;
  int nsup = 0;
  if (iparams != nullptr) {
    nsup = min(max(iparams[row * icolumns + 5], 0), kLogprobMaxSuppressed);
    if (threadIdx.x < nsup) suppressed[threadIdx.x] = iparams[row * icolumns + 6 + threadIdx.x];
  }
  __syncthreads();
  // the slice, scaled; a suppressed id (and, reported, a value that is not finite) takes no part: marked by id -1 below
  float m = -INFINITY;
  bool bad = false;
  for (int j = threadIdx.x; j < n; j += kTopThreads) {
    float v = x[j] / temperature;
    if (!isfinite(v)) {
      bad = true;
      v = -INFINITY;
    }
    for (int k = 0; k < nsup; ++k)
      if (suppressed[k] == lo + j) v = -INFINITY;
    slice[j] = v;
    m = fmaxf(m, v);
  }
  if (bad) publish_error(error, kNonFiniteLogit);
  int none = -1;
  {
    int id = m == -INFINITY ? -1 : 0;
    block_best(m, id, scratch_v, scratch_i);             // (only the value matters here)
    none = id;
  }
  float sum = 0.0f;
  if (none >= 0)
    for (int j = threadIdx.x; j < n; j += kTopThreads)
      if (slice[j] != -INFINITY) sum += expf(slice[j] - m);
  sum = block_sum(sum, scratch_v);
  const size_t part = static_cast<size_t>(row) * slices + sl;
  if (threadIdx.x == 0) {
    part_ms[part * 2] = m;
    part_ms[part * 2 + 1] = sum;
  }
  for (int c = 0; c < count; ++c) {
    float bv = 0.0f;
    int bi = -1;
    for (int j = threadIdx.x; j < n; j += kTopThreads) {
      const float v = slice[j];
      if (v != -INFINITY) keep_better(bv, bi, v, lo + j);
    }
    block_best(bv, bi, scratch_v, scratch_i);
    if (threadIdx.x == 0) {
      part_v[part * count + c] = bv;
      part_i[part * count + c] = bi;
      if (bi >= 0) slice[bi - lo] = -INFINITY;            // taken
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(128)
top_logprobs_merge_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i,
                          const float* __restrict__ part_ms, int slices, int count, int* __restrict__ out_ids,
                          float* __restrict__ out_lps, uint32_t* error) {
  wait_for_prior_kernels();
  launch_dependents();
  __shared__ float cand_v[kTopMaxSlices * kTopLogprobsMax];
  __shared__ int cand_i[kTopMaxSlices * kTopLogprobsMax];
  __shared__ float scratch_v[33];
  __shared__ int scratch_i[33];
  const int row = blockIdx.x;
  const int total = slices * count;
  for (int j = threadIdx.x; j < total; j += blockDim.x) {
    cand_v[j] = part_v[static_cast<size_t>(row) * total + j];
    cand_i[j] = part_i[static_cast<size_t>(row) * total + j];
  }
  float m = -INFINITY;
  for (int sl = threadIdx.x; sl < slices; sl += blockDim.x) m = fmaxf(m, part_ms[(static_cast<size_t>(row) * slices + sl) * 2]);
  {
    int id = m == -INFINITY ? -1 : 0;
    block_best(m, id, scratch_v, scratch_i);
  }
  float sum = 0.0f;
  for (int sl = threadIdx.x; sl < slices; sl += blockDim.x) {
    const float ms = part_ms[(static_cast<size_t>(row) * slices + sl) * 2];
    if (ms != -INFINITY) sum += part_ms[(static_cast<size_t>(row) * slices + sl) * 2 + 1] * expf(ms - m);
  }
  sum = block_sum(sum, scratch_v);
  const float logsumexp = m + logf(sum);
  if (threadIdx.x == 0 && !(sum > 0.0f)) publish_error(error, kNonFiniteLogit);
  for (int c = 0; c < count; ++c) {
    float bv = 0.0f;
    int bi = -1, bj = -1;
    for (int j = threadIdx.x; j < total; j += blockDim.x) {
      if (cand_i[j] < 0) continue;
      if (bi < 0 || cand_v[j] > bv || (cand_v[j] == bv && cand_i[j] < bi)) {
        bv = cand_v[j];
        bi = cand_i[j];
        bj = j;
      }
    }
    block_best(bv, bi, scratch_v, scratch_i);
    if (bj >= 0 && cand_i[bj] == bi) cand_i[bj] = -1;      // taken (ids are unique: one thread holds it)
    if (threadIdx.x == 0) {
      out_ids[static_cast<size_t>(row) * count + c] = bi;
      out_lps[static_cast<size_t>(row) * count + c] = bi >= 0 ? bv - logsumexp : -INFINITY;
    }
    __syncthreads();
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

// How many slices pih_top_logprobs cuts a row of `vocab` logits into, and the 4-byte words of scratch it wants:
// [rows, slices, count] values, the same of ids, [rows, slices, 2] maxima and sums.
extern "C" int pih_top_logprobs_slices(int vocab) {
  int slices = 8;
  while (slices < kTopMaxSlices && (vocab + slices - 1) / slices > kTopSliceFloats) slices *= 2;
  return (vocab + slices - 1) / slices > kTopSliceFloats ? -1 : slices;
}
extern "C" long long pih_top_logprobs_scratch_words(int rows, int vocab, int count) {
  const int slices = pih_top_logprobs_slices(vocab);
  if (slices < 0) return -1;
  return static_cast<long long>(rows) * slices * (2 * count + 2);
}

// out_ids / out_lps [rows, count]: the `count` (1 to 20) most probable ids of every row that are not suppressed, by
// value then id, and their log-probabilities under the row's scaled logits.  fparams / iparams as
// pih_selected_logprob takes them.
extern "C" int pih_top_logprobs(const float* logits, int rows, int vocab, int count, const float* fparams,
                                const int* iparams, int icolumns, int* out_ids, float* out_lps, void* scratch,
                                uint32_t* error, void* stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || count < 1 || count > kTopLogprobsMax || scratch == nullptr ||
      (iparams != nullptr && icolumns < 6 + kLogprobMaxSuppressed))
    return PIH_ERR_BAD_ARGUMENT;
  const int slices = pih_top_logprobs_slices(vocab);
  if (slices < 0 || rows > 65535) return PIH_ERR_UNSUPPORTED;
  const int slice_len = (vocab + slices - 1) / slices;
  const size_t smem = static_cast<size_t>(slice_len) * sizeof(float);
  static size_t smem_set = 0;
  if (smem > 40 * 1024 && smem_set < smem) {
    cudaError_t e = cudaFuncSetAttribute(top_logprobs_slices_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    smem_set = smem;
  }
  float* part_v = static_cast<float*>(scratch);
  int* part_i = reinterpret_cast<int*>(part_v + static_cast<size_t>(rows) * slices * count);
  float* part_ms = reinterpret_cast<float*>(part_i + static_cast<size_t>(rows) * slices * count);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  launch_kernel(top_logprobs_slices_kernel, dim3(slices, rows), dim3(kTopThreads), smem, s, logits, vocab, count,
                slice_len, fparams, iparams, icolumns, part_v, part_i, part_ms, error);
  PIH_LAUNCH_CHECK();
  launch_kernel(top_logprobs_merge_kernel, dim3(rows), dim3(128), 0, s, part_v, part_i, part_ms, slices, count, out_ids,
                out_lps, error);
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
  if (vocab > kSampleCluster * 65536) return PIH_ERR_UNSUPPORTED;      // (the 32-bit sums of a block's part)
  // a block's part of a row in shared memory, if it fits beside the kernel's own
  const int part = (vocab + kSampleCluster - 1) / kSampleCluster;
  int staged_floats = part;
  static long long room = -1;                           // dynamic shared memory that the kernel's own leaves
  if (room < 0) {
    cudaFuncAttributes attr;
    cudaError_t e = cudaFuncGetAttributes(&attr, sample_kernel);
    if (e != cudaSuccess) return static_cast<int>(e);
    room = 227 * 1024 - static_cast<long long>(attr.sharedSizeBytes) - 1024;
  }
  if (static_cast<long long>(part) * 4 > room) staged_floats = 0;
  static int smem_set = 0;
  if (staged_floats * 4 > 40 * 1024 && smem_set < staged_floats * 4) {
    cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, staged_floats * 4);
    if (e != cudaSuccess) return static_cast<int>(e);
    smem_set = staged_floats * 4;
  }
  // Few rows: every cluster finds SMs of its own, and a block of 1024 threads finishes its part sooner (one to eight
  // rows: 56 against 73 us).  More rows: blocks of 512 threads, of which an SM holds two (64 rows: 178 against
  // 277 us; 18 rows: 89 against 111 — 148 SMs hold 16 clusters of eight blocks that want an SM each).
  const int threads = rows <= 8 ? kSampleBlock : kSampleBlock / 2;
  launch_kernel_clustered(sample_kernel, dim3(rows * kSampleCluster), dim3(threads), static_cast<size_t>(staged_floats) * 4,
                          static_cast<cudaStream_t>(stream), static_cast<unsigned>(kSampleCluster), logits, vocab, fparams,
                          iparams, out_tokens, staged_floats, error);
  PIH_LAUNCH_CHECK();
  return 0;
}
