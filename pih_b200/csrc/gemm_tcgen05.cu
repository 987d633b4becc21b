// C[M,N] = A[M,K] . W[N,K]^T in bf16 on the 5th-generation tensor cores:
// tcgen05.mma with the accumulator in tensor memory, operands brought to
// shared memory by TMA (128-byte swizzle), fp32 accumulation, bf16 or fp32
// output rounded once.
//
// The reference runs every product through cuBLASLt
// (src/backend/cuda/gemm_plan.cpp:83-199) and has no kernel of its own.
//
// Two kernels.  gemm_tcgen05_kernel, described here: a tile of C is 128 x BN (BN = 64, 128 or 256); the kernel is
// persistent, one CTA per SM walking over tiles, with two accumulators in tensor memory so that the epilogue of one
// tile overlaps the products of the next.  Warp roles:
//   warp 0      TMA producer: one thread issues the two tile loads of a k-block
//               (A 128 x 64, W BN x 64) into a ring of STAGES buffers;
//   warp 1      allocates tensor memory, then one thread issues the four
//               tcgen05.mma (K = 16 each) of a k-block and commits them to the
//               buffer's "empty" barrier, which frees the buffer when they finish;
//   warps 2-5   epilogue: wait for the accumulator, read it from tensor memory
//               (tcgen05.ld, one row per thread), convert and store.
// Both operands are K-major ("TN"): the natural layout of activations [M,K]
// and weights [N,K].  Rows and columns beyond M, N or K are zero-filled by
// TMA on the way in and masked on the way out, so every size is taken as long
// as K is a multiple of 8 (a TMA row stride must be a multiple of 16 bytes).
//
// Every wait on an mbarrier is bounded; when a bound is hit the kernel records
// kWaitTimedOut, stops waiting, still frees its tensor memory and returns.
// gemm_tcgen05_pair_kernel, described further down: two CTAs of a cluster on one 256 x BN tile (cta_group::2), the
// output through TMA stores; it is the one that the engine uses (gate/up of large prompt portions, SiLU-mul fused).
// Every load of both kernels goes to the shared memory of the CTA that issues it.
#include "ptx.cuh"

namespace pih {

constexpr int GM = 128;          // tile rows (UMMA M)
constexpr int GK = 64;           // k-block: 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
// Shared-memory matrix descriptor of a K-major operand tile stored as rows of 128 bytes with the
// 128-byte swizzle (what TMA writes): 8-row groups are 1024 bytes apart (stride byte offset), the
// leading byte offset is 1 (unused for swizzled K-major), version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);          // start address, bits [0,14)
  desc |= static_cast<uint64_t>(1) << 16;                             // leading byte offset >> 4
  desc |= static_cast<uint64_t>(1024 >> 4) << 32;                     // stride byte offset >> 4
  desc |= static_cast<uint64_t>(1) << 46;                             // version
  desc |= static_cast<uint64_t>(2) << 61;                             // SWIZZLE_128B
  return desc;
}

// Instruction descriptor, kind::f16: fp32 accumulator, bf16 A and B, both K-major, N and M.
__host__ __device__ constexpr uint32_t umma_instr_desc(int m, int n) {
  return (1u << 4)                                  // c_format = F32
         | (1u << 7)                                // a_format = BF16
         | (1u << 10)                               // b_format = BF16
         | (static_cast<uint32_t>(n >> 3) << 17)    // n_dim
         | (static_cast<uint32_t>(m >> 4) << 24);   // m_dim
}

template <int BN, int NSTAGES>
struct GemmSmem {
  alignas(1024) __nv_bfloat16 a[NSTAGES][GM * GK];   // 16 KB per stage
  alignas(1024) __nv_bfloat16 b[NSTAGES][BN * GK];   // BN / 8 KB per stage
  alignas(8) uint64_t full[NSTAGES];
  alignas(8) uint64_t empty[NSTAGES];
  alignas(8) uint64_t accum_full[2];
  alignas(8) uint64_t accum_empty[2];
  uint32_t tmem_base;
};

// 32 consecutive columns of this thread's tensor-memory lane (one row of the accumulator): asked for here,
// in the registers only after tmem_loads_wait().
__device__ __forceinline__ void tmem_load_32_columns_issue(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]),
        "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]),
        "=r"(v[30]), "=r"(v[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_loads_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_load_32_columns(uint32_t taddr, uint32_t (&v)[32]) {
  tmem_load_32_columns_issue(taddr, v);
  tmem_loads_wait();
}

// One chunk of the epilogue: 32 consecutive accumulator columns (from column `col` of the product) of row `row`,
// rounded once and stored.  SWIGLU: the 32 columns are two blocks of 8 gate + 8 up columns and become 16 outputs.
template <typename TC, bool SWIGLU>
__device__ __forceinline__ void store_chunk(const uint32_t (&v)[32], TC* __restrict__ C, int row, int M, int N, int col,
                                            long long ldc) {
  if (SWIGLU) {
    if constexpr (sizeof(TC) == 2) {
      if (row < M && col < N) {                   // N is a multiple of 16, so is col: whole blocks
        TC* dst = C + static_cast<long long>(row) * ldc + col / 2;
        uint32_t packed[8];
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
#pragma unroll
          for (int i = 0; i < 8; i += 2) {
            float o[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const float g = round_to<TC>(__uint_as_float(v[16 * blk + i + e]));
              const float u = round_to<TC>(__uint_as_float(v[16 * blk + 8 + i + e]));
              o[e] = silu_times<TC>(g, u);
            }
            __nv_bfloat162 h = __floats2bfloat162_rn(o[0], o[1]);
            packed[4 * blk + i / 2] = *reinterpret_cast<uint32_t*>(&h);
          }
        }
        const int live = min(2, (N - col) / 16);  // blocks of this chunk that exist
        if (live == 2 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
          reinterpret_cast<uint4*>(dst)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          reinterpret_cast<uint4*>(dst)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        } else {
          for (int j = 0; j < 4 * live; ++j) reinterpret_cast<uint32_t*>(dst)[j] = packed[j];
        }
      }
    }
  } else if (row < M && col < N) {
    TC* dst = C + static_cast<long long>(row) * ldc + col;
    const bool full = col + 32 <= N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
    if (full) {
      if constexpr (sizeof(TC) == 2) {
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
          packed[j] = *reinterpret_cast<uint32_t*>(&h);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
          reinterpret_cast<uint4*>(dst)[j] =
              make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          reinterpret_cast<uint4*>(dst)[j] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
      }
    } else {
      for (int j = 0; j < 32; ++j)
        if (col + j < N) dst[j] = from_float<TC>(__uint_as_float(v[j]));
    }
  }
}

// Persistent: CTA b computes tiles b, b + gridDim.x, ... (tile t = (t % tiles_m, t / tiles_m), so that the
// CTAs that run together share a panel of W in L2).  Two accumulators in tensor memory alternate, so the
// epilogue of one tile overlaps the products of the next.
template <typename TC, int BN, int NSTAGES>
__global__ void __launch_bounds__(192)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    TC* __restrict__ C, int M, int N, int K, long long ldc, uint32_t* error) {
  wait_for_prior_kernels();
  using Smem = GemmSmem<BN, NSTAGES>;
  extern __shared__ unsigned char smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kblocks = (K + GK - 1) / GK;
  const int tiles_m = (M + GM - 1) / GM, tiles_n = (N + BN - 1) / BN;
  const int tiles = tiles_m * tiles_n;
  constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;       // a power of two: BN is 64, 128 or 256

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGES; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sm.accum_full[b], 1);
      mbar_init(&sm.accum_empty[b], 4);          // one arrival per epilogue warp
    }
    mbar_init_fence();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = sm.tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_map(&map_a);
      tma_prefetch_map(&map_w);
      uint32_t it = 0;                           // k-blocks issued so far, over all tiles
      bool alive = true;
      for (int t = blockIdx.x; t < tiles && alive; t += gridDim.x) {
        const int m0 = (t % tiles_m) * GM, n0 = (t / tiles_m) * BN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % NSTAGES;
          const uint32_t round = it / NSTAGES;
          if (round > 0 && !mbar_wait(&sm.empty[s], (round - 1) & 1, error)) {
            alive = false;
            break;
          }
          mbar_expect_tx(&sm.full[s], (GM + BN) * GK * sizeof(__nv_bfloat16));
          tma_load_2d(sm.a[s], &map_a, kb * GK, m0, &sm.full[s]);
          tma_load_2d(sm.b[s], &map_w, kb * GK, n0, &sm.full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_instr_desc(GM, BN);
      uint32_t it = 0, local = 0;
      bool alive = true;
      for (int t = blockIdx.x; t < tiles && alive; t += gridDim.x, ++local) {
        const uint32_t buf = local & 1, use = local >> 1;       // use-th time this accumulator is filled
        if (use > 0 && !mbar_wait(&sm.accum_empty[buf], (use - 1) & 1, error)) break;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t tmem_acc = tmem_base + buf * BN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % NSTAGES;
          if (!mbar_wait(&sm.full[s], (it / NSTAGES) & 1, error)) {
            alive = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const uint32_t a_addr = smem_u32(sm.a[s]), b_addr = smem_u32(sm.b[s]);
#pragma unroll
          for (int k = 0; k < GK / UMMA_K; ++k) {
            const uint64_t adesc = umma_smem_desc(a_addr + k * UMMA_K * 2);
            const uint64_t bdesc = umma_smem_desc(b_addr + k * UMMA_K * 2);
            const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
            asm volatile(
                "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_acc),
                "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
                : "memory");
          }
          // frees the buffer when the MMAs that read it have finished
          asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(
                           smem_u32(&sm.empty[s]))
                       : "memory");
        }
        if (!alive) break;
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(
                         smem_u32(&sm.accum_full[buf]))
                     : "memory");
      }
    }
  } else {
    // epilogue: warp w may touch tensor-memory lanes 32 * (w % 4) .. + 31
    const int quarter = warp & 3;
    uint32_t local = 0;
    for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++local) {
      const uint32_t buf = local & 1, use = local >> 1;
      const int m0 = (t % tiles_m) * GM, n0 = (t / tiles_m) * BN;
      if (!mbar_wait(&sm.accum_full[buf], use & 1, error)) break;
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const int row = m0 + quarter * 32 + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t v[32];
        const uint32_t taddr = tmem_base + buf * BN + (static_cast<uint32_t>(quarter * 32) << 16) + c0;
        tmem_load_32_columns(taddr, v);
        store_chunk<TC, false>(v, C, row, M, N, n0 + c0, ldc);
      }
      // the accumulator may be overwritten once all four epilogue warps have read it
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.accum_empty[buf]);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS));
  }
}

// ---------------------------------------------------------------------------------------------------------
// The same product with PAIRS of SMs on one 256 x BN tile (tcgen05 cta_group::2).  The two CTAs of a cluster
// each hold half of the tile's rows of A (128 x 64 per k-block) and half of its rows of W (BN / 2 x 64), and
// the tensor cores of both SMs read both halves of W: a CTA brings 32 KB per k-block into its shared memory
// for 256 x 256 x 64 of product per pair, where a single CTA on a 128 x 256 tile brings 48 KB for half of
// that — the shared-memory port, which carries the TMA writes and the operand reads, is what bounded the
// single-CTA kernel (tensor pipe 52 % busy).  Every load goes to the shared memory of the CTA that issues it.
//   CTA 0 of the pair (the leader): its MMA thread issues every tcgen05.mma for both SMs, and commits them
//       to the "empty" barrier of the stage and to the "accumulator full" barrier in BOTH CTAs;
//   both CTAs: the producer thread loads the CTA's own halves into its own ring; the loads of both CTAs
//       complete on the LEADER's "full" barrier, which expects the bytes of both;
//   both CTAs: eight epilogue warps read the CTA's 128 rows of the accumulator from its own tensor memory
//       (a quarter of the rows and half of the columns each); each tells the leader's "accumulator empty"
//       barrier (16 arrivals) when it has read it.
// A cluster barrier after the set-up (no CTA signals a barrier that is not initialised) and one before the
// tensor memory is freed (no CTA leaves while the other may still read its shared memory or signal it).
// SWIGLU: the rows of W (columns of the product) come in blocks of 16 = 8 gate columns + their 8 up columns, and
// the epilogue writes out[m, 8 b + i] = round(silu(round(g)) * round(u)) for block b — C is [M, N / 2] — with the
// roundings of the separate kernels (the product's bf16 output, then SiLU-mul): the gate/up product of a prompt
// portion never writes its [M, 2 I] result to memory.
template <int BN, int NSTAGES>
struct PairSmem {
  alignas(1024) __nv_bfloat16 a[NSTAGES][GM * GK];          // this CTA's 128 rows of A
  alignas(1024) __nv_bfloat16 b[NSTAGES][(BN / 2) * GK];    // this CTA's BN / 2 rows of W
  alignas(1024) unsigned char stage[8][32 * 128];           // per epilogue warp: 32 rows of 128 bytes on their way out
  alignas(8) uint64_t full[NSTAGES];                        // used in the leader
  alignas(8) uint64_t empty[NSTAGES];
  alignas(8) uint64_t accum_full[2];
  alignas(8) uint64_t accum_empty[2];                       // used in the leader
  uint32_t tmem_base;
};

__device__ __forceinline__ uint32_t pair_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// the address that `local` (in this CTA's shared memory) has in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t address_in_cta(const void* local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
  return remote;
}
__device__ __forceinline__ void pair_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA tile load of a CTA pair: into this CTA's shared memory, completing on a barrier of either CTA
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], "
      "[%4];\n" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar_cluster_addr)
      : "memory");
}
// the barrier (an address in the cluster's shared memory) learns when every MMA issued so far has finished
__device__ __forceinline__ void pair_commit(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar_cluster_addr)
               : "memory");
}

// 32 accumulator columns of one row as they are stored: kChunkWords 32-bit words (SWIGLU: 16 bf16 outputs of two
// blocks of 8 gate + 8 up columns; else 32 bf16 or 32 floats), rounded once.
template <typename TC, bool SWIGLU>
constexpr int kChunkWords = SWIGLU ? 8 : (sizeof(TC) == 2 ? 16 : 32);

template <typename TC, bool SWIGLU>
__device__ __forceinline__ void convert_chunk(const uint32_t (&v)[32], uint32_t (&w)[kChunkWords<TC, SWIGLU>]) {
  if constexpr (SWIGLU) {
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
#pragma unroll
      for (int i = 0; i < 8; i += 2) {
        float o[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float g = round_to<TC>(__uint_as_float(v[16 * blk + i + e]));
          const float u = round_to<TC>(__uint_as_float(v[16 * blk + 8 + i + e]));
          o[e] = silu_times<TC>(g, u);
        }
        __nv_bfloat162 h = __floats2bfloat162_rn(o[0], o[1]);
        w[4 * blk + i / 2] = *reinterpret_cast<uint32_t*>(&h);
      }
    }
  } else if constexpr (sizeof(TC) == 2) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
      w[j] = *reinterpret_cast<uint32_t*>(&h);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) w[j] = v[j];
  }
}

// TMA store of a box from this CTA's shared memory (written by ordinary stores: fence first), as one bulk group
__device__ __forceinline__ void fence_smem_for_tma() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y, const void* smem_src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];\n" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(x), "r"(y), "r"(smem_u32(smem_src))
               : "memory");
  asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
}
__device__ __forceinline__ void tma_stores_have_read() { asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory"); }

template <typename TC, int BN, int NSTAGES, bool SWIGLU>
__global__ void __launch_bounds__(320)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                         const __grid_constant__ CUtensorMap map_c, int store_by_tma, TC* __restrict__ C, int M, int N,
                         int K, long long ldc, uint32_t* error) {
  using Smem = PairSmem<BN, NSTAGES>;
  extern __shared__ unsigned char smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = pair_rank();
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int kblocks = (K + GK - 1) / GK;
  const int tiles_m = (M + 2 * GM - 1) / (2 * GM), tiles_n = (N + BN - 1) / BN;
  const int tiles = tiles_m * tiles_n;
  constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;       // a power of two: BN is 128 or 256

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGES; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sm.accum_full[b], 1);
      mbar_init(&sm.accum_empty[b], 16);         // one arrival per epilogue warp of both CTAs
    }
    mbar_init_fence();
  }
  if (warp == 1) {                               // the same warp of both CTAs, together
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::);
  }
  if (threadIdx.x == 32) {
    tma_prefetch_map(&map_a);
    tma_prefetch_map(&map_w);
    tma_prefetch_map(&map_c);
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  pair_sync();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = sm.tmem_base;
  wait_for_prior_kernels();                      // all of the above ran beside the end of the kernel before this one

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;                           // k-blocks issued so far, over all tiles
      bool alive = true;
      for (int t = pair; t < tiles && alive; t += pairs) {
        const int m0 = (t % tiles_m) * 2 * GM + static_cast<int>(rank) * GM;
        const int n0 = (t / tiles_m) * BN + static_cast<int>(rank) * (BN / 2);
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % NSTAGES;
          const uint32_t round = it / NSTAGES;
          if (round > 0 && !mbar_wait(&sm.empty[s], (round - 1) & 1, error)) {
            alive = false;
            break;
          }
          if (rank == 0) mbar_expect_tx(&sm.full[s], 2 * (GM + BN / 2) * GK * sizeof(__nv_bfloat16));
          const uint32_t full_of_leader = address_in_cta(&sm.full[s], 0);
          tma_load_2d_pair(sm.a[s], &map_a, kb * GK, m0, full_of_leader);
          tma_load_2d_pair(sm.b[s], &map_w, kb * GK, n0, full_of_leader);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_instr_desc(2 * GM, BN);
      uint32_t it = 0, local = 0;
      bool alive = true;
      for (int t = pair; t < tiles && alive; t += pairs, ++local) {
        const uint32_t buf = local & 1, use = local >> 1;       // use-th time this accumulator is filled
        if (use > 0 && !mbar_wait(&sm.accum_empty[buf], (use - 1) & 1, error)) break;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t tmem_acc = tmem_base + buf * BN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % NSTAGES;
          if (!mbar_wait(&sm.full[s], (it / NSTAGES) & 1, error)) {
            alive = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const uint32_t a_addr = smem_u32(sm.a[s]), b_addr = smem_u32(sm.b[s]);
#pragma unroll
          for (int k = 0; k < GK / UMMA_K; ++k) {
            const uint64_t adesc = umma_smem_desc(a_addr + k * UMMA_K * 2);
            const uint64_t bdesc = umma_smem_desc(b_addr + k * UMMA_K * 2);
            const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
            asm volatile(
                "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_acc),
                "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
                : "memory");
          }
          // frees the buffer in both CTAs when the MMAs that read it have finished
          pair_commit(address_in_cta(&sm.empty[s], 0));
          pair_commit(address_in_cta(&sm.empty[s], 1));
        }
        if (!alive) break;
        pair_commit(address_in_cta(&sm.accum_full[buf], 0));
        pair_commit(address_in_cta(&sm.accum_full[buf], 1));
      }
    }
  } else {
    // epilogue, eight warps: warp w may touch tensor-memory lanes 32 * (w % 4) .. + 31; warps 2-5 take the left
    // half of the tile's columns, warps 6-9 the right half
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    uint32_t local = 0;
    for (int t = pair; t < tiles; t += pairs, ++local) {
      const uint32_t buf = local & 1, use = local >> 1;
      const int m0 = (t % tiles_m) * 2 * GM + static_cast<int>(rank) * GM, n0 = (t / tiles_m) * BN;
      if (!mbar_wait(&sm.accum_full[buf], use & 1, error)) break;
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const int row = m0 + quarter * 32 + lane;
      const uint32_t tmem_row = tmem_base + buf * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      constexpr int CHUNKS = BN / 64;                    // chunks of 32 accumulator columns of this warp's half
      const int c_first = half * (BN / 2);
      if (store_by_tma) {
        // Rows leave as 128-byte pieces: the warp's 32 rows of 32 output words are put into shared memory as TMA
        // wants them (16-byte chunk c of row r at chunk c ^ (r & 7): no bank is hit twice) and one thread sends the
        // box; TMA drops what lies beyond M or the last column.  The next box waits until this one has been read.
        // The next chunk is on its way out of tensor memory while this one is converted.
        constexpr int WORDS = kChunkWords<TC, SWIGLU>;
        constexpr int PER_BOX = 32 / WORDS;              // chunks of 32 accumulator columns in a box
        static_assert(CHUNKS % PER_BOX == 0, "a warp's half of the tile is whole boxes");
        unsigned char* stage = sm.stage[warp - 2];
        uint32_t v[2][32];
        tmem_load_32_columns_issue(tmem_row + c_first, v[0]);
#pragma unroll
        for (int i = 0; i < CHUNKS; ++i) {
          const int c0 = c_first + 32 * i;
          tmem_loads_wait();
          if (i + 1 < CHUNKS) tmem_load_32_columns_issue(tmem_row + c0 + 32, v[(i + 1) & 1]);
          uint32_t w[WORDS];
          convert_chunk<TC, SWIGLU>(v[i & 1], w);
          const int sub = i % PER_BOX;
          if (sub == 0) {
            if (lane == 0) tma_stores_have_read();
            __syncwarp();
          }
#pragma unroll
          for (int j = 0; j < WORDS / 4; ++j) {
            const int chunk = sub * (WORDS / 4) + j;
            *reinterpret_cast<uint4*>(stage + lane * 128 + ((chunk ^ (lane & 7)) << 4)) =
                make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
          }
          if (sub == PER_BOX - 1) {
            fence_smem_for_tma();
            __syncwarp();
            const int acc_col = n0 + c0 - 32 * (PER_BOX - 1);
            const int x = SWIGLU ? acc_col / 2 : acc_col, y = m0 + quarter * 32;
            if (lane == 0 && y < M && acc_col < N) tma_store_2d(&map_c, x, y, stage);
          }
        }
      } else {
#pragma unroll 1
        for (int i = 0; i < CHUNKS; ++i) {
          uint32_t v[32];
          tmem_load_32_columns(tmem_row + c_first + 32 * i, v);
          store_chunk<TC, SWIGLU>(v, C, row, M, N, n0 + c_first + 32 * i, ldc);
        }
      }
      // the accumulator may be overwritten once the epilogue warps of both CTAs have read it
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        const uint32_t bar = address_in_cta(&sm.accum_empty[buf], 0);
        asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(bar) : "memory");
      }
    }
    if (lane == 0) tma_stores_have_read();       // the boxes have left shared memory (no group pends where none was sent)
  }
  __syncwarp();                                  // (the barrier below wants whole warps)
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  pair_sync();                                   // nothing of either CTA is in use any more
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS));
  }
}

// 2-D bf16 tensor [rows, cols] with a row stride of ld elements; box = box_rows x 64 columns, 128-byte swizzle.
static bool make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
  EncodeTiledFn fn = encode_tiled();
  if (fn == nullptr) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * sizeof(__nv_bfloat16)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(GK), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The output [rows, cols] of 2- or 4-byte elements with a row stride of ld elements; box = 32 rows of 128 bytes,
// 128-byte swizzle.
static bool make_out_map(CUtensorMap* map, void* base, long long rows, long long cols, long long ld, int elem_bytes) {
  EncodeTiledFn fn = encode_tiled();
  if (fn == nullptr) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * elem_bytes};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / elem_bytes), 32u};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims,
            strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace pih

using namespace pih;

// out_dtype: PIH_BF16 or PIH_F32.  Returns PIH_ERR_UNSUPPORTED when the operands cannot be described
// to TMA (K or a row stride not a multiple of 8 elements, a base not 16-byte aligned): the caller then
// uses another product.
template <typename TC, int BN, int NSTAGES>
static int launch_gemm(const CUtensorMap& map_a, const CUtensorMap& map_w, void* C, int M, int N, int K,
                       long long ldc, uint32_t* error, int sms, cudaStream_t s) {
  const int smem = static_cast<int>(sizeof(GemmSmem<BN, NSTAGES>)) + 1024;
  static bool configured = false;                     // per instance
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<TC, BN, NSTAGES>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  const long long tiles = static_cast<long long>((M + GM - 1) / GM) * ((N + BN - 1) / BN);
  const int grid = static_cast<int>(tiles < sms ? tiles : sms);
  launch_kernel(gemm_tcgen05_kernel<TC, BN, NSTAGES>, dim3(grid), dim3(192), smem, s, map_a, map_w, static_cast<TC*>(C), M, N, K, ldc, error);
  PIH_LAUNCH_CHECK();
  return 0;
}

template <typename TC>
static int launch_gemm_bn(int bn, const CUtensorMap& map_a, const CUtensorMap& map_w, void* C, int M, int N, int K,
                          long long ldc, uint32_t* error, int sms, cudaStream_t s) {
  if (bn == 256) return launch_gemm<TC, 256, 4>(map_a, map_w, C, M, N, K, ldc, error, sms, s);
  if (bn == 128) return launch_gemm<TC, 128, 6>(map_a, map_w, C, M, N, K, ldc, error, sms, s);
  return launch_gemm<TC, 64, 8>(map_a, map_w, C, M, N, K, ldc, error, sms, s);
}

// out_dtype: PIH_BF16 or PIH_F32.  tile_n: 64, 128 or 256 columns per tile, or 0 to let the entry point
// choose (the widest tile that still gives every SM work).  Returns PIH_ERR_UNSUPPORTED when the operands
// cannot be described to TMA (K or a row stride not a multiple of 8 elements, a base not 16-byte aligned):
// the caller then uses another product.
extern "C" int pih_gemm_tcgen05(int out_dtype, const void* A, const void* W, void* C, int M, int N, int K,
                                long long lda, long long ldw, long long ldc, int tile_n, uint32_t* error,
                                void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (tile_n != 0 && tile_n != 64 && tile_n != 128 && tile_n != 256)) return PIH_ERR_BAD_ARGUMENT;
  if (K % 8 || lda % 8 || ldw % 8 || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(W) & 15))
    return PIH_ERR_UNSUPPORTED;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  int bn = tile_n;
  if (bn == 0) {
    // fewest "waves x (tile width + fixed cost)" wins
    const long long tiles_m = (M + GM - 1) / GM;
    long long best = -1;
    for (int cand = 64; cand <= 256; cand *= 2) {
      const long long tiles = tiles_m * ((N + cand - 1) / cand);
      const long long cost = ((tiles + sms - 1) / sms) * (cand + 64);
      if (best < 0 || cost <= best) {
        best = cost;
        bn = cand;
      }
    }
  }
  CUtensorMap map_a, map_w;
  if (!make_map(&map_a, A, M, K, lda, GM) || !make_map(&map_w, W, N, K, ldw, bn)) return PIH_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (out_dtype == PIH_BF16) return launch_gemm_bn<__nv_bfloat16>(bn, map_a, map_w, C, M, N, K, ldc, error, sms, s);
  if (out_dtype == PIH_F32) return launch_gemm_bn<float>(bn, map_a, map_w, C, M, N, K, ldc, error, sms, s);
  return PIH_ERR_BAD_ARGUMENT;
}

template <typename TC, int BN, int NSTAGES, bool SWIGLU>
static int launch_pair(const CUtensorMap& map_a, const CUtensorMap& map_w, const CUtensorMap& map_c, int store_by_tma,
                       void* C, int M, int N, int K, long long ldc, uint32_t* error, cudaStream_t s) {
  const int smem = static_cast<int>(sizeof(PairSmem<BN, NSTAGES>)) + 1024;
  static int max_pairs = 0;                           // per instance: clusters of two that the device holds at once
  auto kernel = gemm_tcgen05_pair_kernel<TC, BN, NSTAGES, SWIGLU>;
  if (max_pairs == 0) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2);
    cfg.blockDim = dim3(320);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr = {};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kernel, &cfg);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (n <= 0) return PIH_ERR_UNSUPPORTED;
    max_pairs = n;
  }
  const long long tiles = static_cast<long long>((M + 2 * GM - 1) / (2 * GM)) * ((N + BN - 1) / BN);
  const int pairs = static_cast<int>(tiles < max_pairs ? tiles : max_pairs);
  launch_kernel_clustered(kernel, dim3(2 * pairs), dim3(320), smem, s, 2u, map_a, map_w, map_c, store_by_tma,
                          static_cast<TC*>(C), M, N, K, ldc, error);
  PIH_LAUNCH_CHECK();
  return 0;
}

// The product on pairs of SMs (256 x tile_n tiles, tile_n 128 or 256; 0: 256).  swiglu != 0: W holds blocks of
// 8 gate rows followed by their 8 up rows (N a multiple of 16), C is [M, N / 2] and bf16, the tile 256 wide.
extern "C" int pih_gemm_tcgen05_pair(int out_dtype, const void* A, const void* W, void* C, int M, int N, int K,
                                     long long lda, long long ldw, long long ldc, int tile_n, int swiglu,
                                     uint32_t* error, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (tile_n != 0 && tile_n != 128 && tile_n != 256)) return PIH_ERR_BAD_ARGUMENT;
  if (swiglu && out_dtype != PIH_BF16) return PIH_ERR_BAD_ARGUMENT;
  if (K % 8 || lda % 8 || ldw % 8 || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(W) & 15))
    return PIH_ERR_UNSUPPORTED;
  if (swiglu && (N % 16 || (reinterpret_cast<uintptr_t>(C) & 3) || ldc % 2)) return PIH_ERR_UNSUPPORTED;
  const int bn = tile_n != 0 && !swiglu ? tile_n : 256;
  CUtensorMap map_a, map_w;
  if (!make_map(&map_a, A, M, K, lda, GM) || !make_map(&map_w, W, N, K, ldw, bn / 2)) return PIH_ERR_UNSUPPORTED;
  // the output leaves through TMA, in boxes of 32 rows of 128 bytes, when it can be described to it
  const long long out_cols = swiglu ? N / 2 : N;
  const int out_bytes = out_dtype == PIH_F32 ? 4 : 2;
  CUtensorMap map_c = {};
  const int store_by_tma = (reinterpret_cast<uintptr_t>(C) & 15) == 0 && (ldc * out_bytes) % 16 == 0 &&
                           make_out_map(&map_c, C, M, out_cols, ldc, out_bytes);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define PIH_PAIR(TC, SW)                                                                                    \
  (bn == 256 ? launch_pair<TC, 256, 6, SW>(map_a, map_w, map_c, store_by_tma, C, M, N, K, ldc, error, s)     \
             : launch_pair<TC, 128, 8, SW>(map_a, map_w, map_c, store_by_tma, C, M, N, K, ldc, error, s))
  if (swiglu)                                           // (its boxes of 64 outputs want the wide tile)
    return launch_pair<__nv_bfloat16, 256, 6, true>(map_a, map_w, map_c, store_by_tma, C, M, N, K, ldc, error, s);
  if (out_dtype == PIH_BF16) return PIH_PAIR(__nv_bfloat16, false);
  if (out_dtype == PIH_F32) return PIH_PAIR(float, false);
#undef PIH_PAIR
  return PIH_ERR_BAD_ARGUMENT;
}

// Where the gate/up product of a SwiGLU feed-forward runs on pairs of SMs with SiLU-mul in its epilogue instead
// of the library's product followed by the SiLU-mul kernel: from g_pair_swiglu_min_rows rows (0: never) when the
// 256 x 256 tiles fill the rounds of the device's SM pairs to four fifths at least.  Measured on [rows, 1024]
// by [6144, 1024]: 20.5 against 20.9 us at 1536 rows, 26.9 against 27.7 at 2048, 46.2 against 51.7 at 4096, 79.9
// against 95.2 at 8192 — and 19.6 against 16.7 at 1024 rows, whose 96 tiles fill two rounds of 74 pairs to 65 %.
static int g_pair_swiglu_min_rows = 1536;
static int g_pair_swiglu_min_fill = 80;     // per cent of the last round's SM pairs that must have a tile

// min_fill_percent < 0 leaves the fill rule as it is.  Returns the previous row count.
extern "C" int pih_set_pair_swiglu_rule(int min_rows, int min_fill_percent) {
  const int before = g_pair_swiglu_min_rows;
  g_pair_swiglu_min_rows = min_rows > 0 ? min_rows : 0;
  if (min_fill_percent >= 0) g_pair_swiglu_min_fill = min_fill_percent > 100 ? 100 : min_fill_percent;
  return before;
}

extern "C" int pih_pair_swiglu_wanted(int rows, int n) {
  if (g_pair_swiglu_min_rows <= 0 || rows < g_pair_swiglu_min_rows || n <= 0) return 0;
  static int pairs = 0;
  if (pairs == 0) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    pairs = sms >= 2 ? sms / 2 : 74;
  }
  const long long tiles = static_cast<long long>((rows + 2 * GM - 1) / (2 * GM)) * ((n + 255) / 256);
  const long long rounds = (tiles + pairs - 1) / pairs;
  return 100 * tiles >= static_cast<long long>(g_pair_swiglu_min_fill) * rounds * pairs ? 1 : 0;
}

