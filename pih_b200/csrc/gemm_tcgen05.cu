// C[M,N] = A[M,K] . W[N,K]^T in bf16 on the 5th-generation tensor cores:
// tcgen05.mma with the accumulator in tensor memory, operands brought to
// shared memory by TMA (128-byte swizzle), fp32 accumulation, bf16 or fp32
// output rounded once.
//
// The reference runs every product through cuBLASLt
// (src/backend/cuda/gemm_plan.cpp:83-199) and has no kernel of its own.
//
// A tile of C is 128 x BN (BN = 64, 128 or 256); the kernel is persistent, one CTA per SM
// walking over tiles, with two accumulators in tensor memory so that the epilogue of one
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
// No cluster launch and no multicast are used.
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

// Persistent: CTA b computes tiles b, b + gridDim.x, ... (tile t = (t % tiles_m, t / tiles_m), so that the
// CTAs that run together share a panel of W in L2).  Two accumulators in tensor memory alternate, so the
// epilogue of one tile overlaps the products of the next.
// SWIGLU: the rows of W (columns of the product) come in blocks of 16 = 8 gate columns + their 8 up columns, and
// the epilogue writes out[m, 8 b + i] = round(silu(round(g)) * round(u)) for block b — C is [M, N / 2] — with the
// roundings of the separate kernels (the product's bf16 output, then SiLU-mul): the gate/up product of a prompt
// portion never writes its [M, 2 I] result to memory.
template <typename TC, int BN, int NSTAGES, bool SWIGLU>
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
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
        if (SWIGLU) {
          if constexpr (sizeof(TC) == 2) {
            if (row < M && n0 + c0 < N) {                   // N is a multiple of 16, so is c0: whole blocks
              TC* dst = C + static_cast<long long>(row) * ldc + (n0 + c0) / 2;
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
              const int live = min(2, (N - (n0 + c0)) / 16);  // blocks of this chunk that exist
              if (live == 2 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                reinterpret_cast<uint4*>(dst)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                reinterpret_cast<uint4*>(dst)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
              } else {
                for (int j = 0; j < 4 * live; ++j) reinterpret_cast<uint32_t*>(dst)[j] = packed[j];
              }
            }
          }
        } else if (row < M && n0 + c0 < N) {
          TC* dst = C + static_cast<long long>(row) * ldc + n0 + c0;
          const bool full = n0 + c0 + 32 <= N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
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
              if (n0 + c0 + j < N) dst[j] = from_float<TC>(__uint_as_float(v[j]));
          }
        }
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

}  // namespace pih

using namespace pih;

// out_dtype: PIH_BF16 or PIH_F32.  Returns PIH_ERR_UNSUPPORTED when the operands cannot be described
// to TMA (K or a row stride not a multiple of 8 elements, a base not 16-byte aligned): the caller then
// uses another product.
template <typename TC, int BN, int NSTAGES, bool SWIGLU = false>
static int launch_gemm(const CUtensorMap& map_a, const CUtensorMap& map_w, void* C, int M, int N, int K,
                       long long ldc, uint32_t* error, int sms, cudaStream_t s) {
  const int smem = static_cast<int>(sizeof(GemmSmem<BN, NSTAGES>)) + 1024;
  static bool configured = false;                     // per instance
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<TC, BN, NSTAGES, SWIGLU>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  const long long tiles = static_cast<long long>((M + GM - 1) / GM) * ((N + BN - 1) / BN);
  const int grid = static_cast<int>(tiles < sms ? tiles : sms);
  launch_kernel(gemm_tcgen05_kernel<TC, BN, NSTAGES, SWIGLU>, dim3(grid), dim3(192), smem, s, map_a, map_w, static_cast<TC*>(C), M, N, K, ldc, error);
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

// The gate/up product of a SwiGLU feed-forward with SiLU-mul in its epilogue (bf16): W [N, K] holds blocks of 8
// gate rows followed by their 8 up rows (N a multiple of 16), C is [M, N / 2] with row stride ldc.
extern "C" int pih_gemm_tcgen05_swiglu(const void* A, const void* W, void* C, int M, int N, int K, long long lda,
                                       long long ldw, long long ldc, int tile_n, uint32_t* error, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (tile_n != 0 && tile_n != 128 && tile_n != 256)) return PIH_ERR_BAD_ARGUMENT;
  if (N % 16 || K % 8 || lda % 8 || ldw % 8 || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(W) & 15) || (reinterpret_cast<uintptr_t>(C) & 3) || ldc % 2)
    return PIH_ERR_UNSUPPORTED;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  const int bn = tile_n != 0 ? tile_n : 256;
  CUtensorMap map_a, map_w;
  if (!make_map(&map_a, A, M, K, lda, GM) || !make_map(&map_w, W, N, K, ldw, bn)) return PIH_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (bn == 256) return launch_gemm<__nv_bfloat16, 256, 4, true>(map_a, map_w, C, M, N, K, ldc, error, sms, s);
  return launch_gemm<__nv_bfloat16, 128, 6, true>(map_a, map_w, C, M, N, K, ldc, error, sms, s);
}
