// Products with few rows (decode: 1..16 tokens): out[M,N] = act[M,K] . W[N,K]^T, bound by reading W once.
//
// The reference pads every decode step to 4096 rows and calls cuBLASLt for each of q, k, v, o, gate, up and
// down (plugins/model-qwen3/nvidia_qwen3_bf16_engine.cpp:391-392; src/backend/cuda/gemm_plan.cpp:192-197),
// with RMSNorm, residual add and SiLU-mul as kernels of their own between them
// (kernels/cuda/qwen_bf16_primitives.cu:264-324).  Here one kernel streams the weight rows once and does
// the small work around the product itself:
//
//   prologue   optional residual add (h <- round(h + delta), written back once) and RMSNorm of the M rows,
//              recomputed by every CTA from the 2 KB rows (cheaper than a kernel of its own and a round trip):
//              a warp per row, all of a lane's loads issued together, the squares summed in registers — one
//              trip to memory, one warp reduction, one barrier (a loop that loaded, added and stored chunk by
//              chunk cost 3 us per product, more than the separate norm kernel it replaced);
//   product    mma.sync m16n8k16 with the TOKENS as the 16-row operand and 8 weight rows as the 8-column
//              operand, so a warp needs only 8 weight rows; each thread reads 16 contiguous bytes of a weight
//              row per 32-wide k block (the k order inside a block is permuted the same way for both operands,
//              which a dot product does not notice); the eight warps of a CTA take every eighth k block and
//              their partial sums are added in a fixed order; the kernel is persistent (two CTAs per SM walk
//              over the weight tiles) so the prologue runs once per CTA and weight loads stay in flight;
//   epilogue   store, or SwiGLU when the CTA's 16 weight rows are 8 gate rows followed by their 8 up rows:
//              out = round(silu(round(g)) * round(u))  (rounding places of the separate kernels).
//
// A row's result does not depend on the other rows of the batch.
#include "common.cuh"

namespace pih {

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_nc16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

constexpr int SK_WARPS = 8;
constexpr int SK_THREADS = SK_WARPS * 32;
constexpr int SK_UN = 4;                 // k blocks in flight per warp unless the product has a long k

// MR: rows of the token operand kept in shared memory (8 or 16).  TILES: 8-row weight tiles per warp (1 or 2).
// UN: k blocks (of 32) whose weight loads a warp keeps in flight.
// Persistent: a CTA prepares the token rows once and then walks over weight tiles blockIdx.x, + gridDim.x, ...
template <int MR, int TILES, int UN, bool NORM, bool SWIGLU, typename NW, typename OT>
__global__ void __launch_bounds__(SK_THREADS)
skinny_gemm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                   __nv_bfloat16* __restrict__ x_out, const NW* __restrict__ norm_w, float eps,
                   const __nv_bfloat16* __restrict__ W, OT* __restrict__ out, int M, int N, int K,
                   long long ldx, long long ldw, long long ldo) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int LDS = K + 8;                                   // padded row: 16-byte loads of 8 rows hit 8 bank groups
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);         // [MR][LDS]
  float* red = reinterpret_cast<float*>(xs + MR * LDS);                   // [SK_WARPS][TILES][16 * 8]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, q = lane & 3;
  const int kblocks = K / 32;
  const int ntiles = (N + 8 * TILES - 1) / (8 * TILES);

  uint4 wv[UN][TILES];
  auto issue = [&](int tile, int first_block) {            // weight loads of k blocks first_block, + WARPS, ...
#pragma unroll
    for (int t = 0; t < TILES; ++t) {
      const int row = min(tile * 8 * TILES + t * 8 + gid, N - 1);
      const __nv_bfloat16* wrow = W + static_cast<long long>(row) * ldw + 8 * q;
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        const int b = first_block + SK_WARPS * u;
        wv[u][t] = (b < kblocks) ? ldg_nc16(wrow + b * 32) : make_uint4(0, 0, 0, 0);
      }
    }
  };
  int tile = blockIdx.x;
  // neither the weight stream nor the norm weights wait for the prologue or for the kernel before this one
  // (no kernel writes weights): the first loads are in flight while that kernel's last blocks finish
  issue(tile, warp);
  const int chunks = K / 8;                                // 16-byte chunks of a token row
  constexpr int NWV = 8 * sizeof(NW) / 16;                 // 16-byte loads per 8 norm weights
  uint4 wpre[4][NWV];                                      // norm weights of the lane's first four chunks
  if (NORM) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = lane + 32 * j;
#pragma unroll
      for (int v = 0; v < NWV; ++v)
        wpre[j][v] = c < chunks ? ldg_nc16(reinterpret_cast<const uint4*>(norm_w + c * 8) + v) : make_uint4(0, 0, 0, 0);
    }
  }
  wait_for_prior_kernels();

  // prologue, once per block: warp w prepares token rows w, w + 8.  A lane takes chunks lane, lane + 32, ...,
  // four at a time with their loads issued together; the residual sum is rounded and kept (one block writes
  // it out), its squares are summed on the way, and the normed row replaces it in shared memory.
  for (int row = warp; row < MR; row += SK_WARPS) {
    __nv_bfloat16* xrow = xs + row * LDS;
    if (row >= M) {
      for (int c = lane; c < chunks; c += 32) *reinterpret_cast<uint4*>(xrow + c * 8) = make_uint4(0, 0, 0, 0);
      continue;
    }
    float ss = 0.0f;
    for (int c0 = 0; c0 < chunks; c0 += 128) {
      uint4 v[4], d[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = c0 + lane + 32 * j;
        v[j] = d[j] = make_uint4(0, 0, 0, 0);
        if (c < chunks) {
          v[j] = *reinterpret_cast<const uint4*>(x + row * ldx + c * 8);
          if (delta != nullptr) d[j] = *reinterpret_cast<const uint4*>(delta + row * ldx + c * 8);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = c0 + lane + 32 * j;
        if (c >= chunks) continue;
        __nv_bfloat16* ve = reinterpret_cast<__nv_bfloat16*>(&v[j]);
        if (delta != nullptr) {
          const __nv_bfloat16* de = reinterpret_cast<const __nv_bfloat16*>(&d[j]);
#pragma unroll
          for (int e = 0; e < 8; ++e) ve[e] = __float2bfloat16_rn(__bfloat162float(ve[e]) + __bfloat162float(de[e]));
          // the sum goes to a buffer of its own: other blocks are still reading x
          if (blockIdx.x == 0) *reinterpret_cast<uint4*>(x_out + row * ldx + c * 8) = v[j];
        }
        if (NORM) {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float f = __bfloat162float(ve[e]);
            ss += f * f;
          }
        }
        *reinterpret_cast<uint4*>(xrow + c * 8) = v[j];
      }
    }
    if (NORM) {
      ss = warp_sum(ss);
      const float scale = 1.0f / sqrtf(ss / static_cast<float>(K) + eps);
      for (int c0 = 0; c0 < chunks; c0 += 128) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int c = c0 + lane + 32 * j;
          if (c >= chunks) continue;
          uint4 wq[NWV];
#pragma unroll
          for (int u = 0; u < NWV; ++u)
            wq[u] = c0 == 0 ? wpre[j][u] : ldg_nc16(reinterpret_cast<const uint4*>(norm_w + c * 8) + u);
          const NW* we = reinterpret_cast<const NW*>(wq);
          uint4 v = *reinterpret_cast<const uint4*>(xrow + c * 8);    // the lane's own store
          __nv_bfloat16* ve = reinterpret_cast<__nv_bfloat16*>(&v);
#pragma unroll
          for (int e = 0; e < 8; ++e)
            ve[e] = __float2bfloat16_rn((__bfloat162float(ve[e]) * scale) * to_float<NW>(we[e]));
          *reinterpret_cast<uint4*>(xrow + c * 8) = v;
        }
      }
    }
  }
  __syncthreads();

  const __nv_bfloat16* xa = xs + gid * LDS + 8 * q;                       // tokens gid (and gid + 8 when MR = 16)
  for (; tile < ntiles; tile += gridDim.x) {
    const int n0 = tile * 8 * TILES;
    float acc[TILES][4];
#pragma unroll
    for (int t = 0; t < TILES; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.0f;
    for (int kb = warp; kb < kblocks; kb += SK_WARPS * UN) {
      uint4 cur[UN][TILES];
#pragma unroll
      for (int u = 0; u < UN; ++u)
#pragma unroll
        for (int t = 0; t < TILES; ++t) cur[u][t] = wv[u][t];
      // the next batch of weight loads — of this tile, or the first of the CTA's next tile — before this one is used
      const int nb = kb + SK_WARPS * UN;
      if (nb < kblocks) issue(tile, nb);
      else if (tile + gridDim.x < ntiles) issue(tile + gridDim.x, warp);
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        const int b = kb + SK_WARPS * u;
        if (b >= kblocks) break;
        const uint4 xlo = *reinterpret_cast<const uint4*>(xa + b * 32);
        uint4 xhi = make_uint4(0, 0, 0, 0);
        if (MR == 16) xhi = *reinterpret_cast<const uint4*>(xa + 8 * LDS + b * 32);
#pragma unroll
        for (int t = 0; t < TILES; ++t) {
          mma16816(acc[t], xlo.x, xhi.x, xlo.y, xhi.y, cur[u][t].x, cur[u][t].y);
          mma16816(acc[t], xlo.z, xhi.z, xlo.w, xhi.w, cur[u][t].z, cur[u][t].w);
        }
      }
    }
    // the warps' partial sums, added in warp order
#pragma unroll
    for (int t = 0; t < TILES; ++t) {
      float* r = red + (warp * TILES + t) * 128;
      r[gid * 8 + q * 2] = acc[t][0];
      r[gid * 8 + q * 2 + 1] = acc[t][1];
      r[(gid + 8) * 8 + q * 2] = acc[t][2];
      r[(gid + 8) * 8 + q * 2 + 1] = acc[t][3];
    }
    __syncthreads();
    if (SWIGLU) {
      // tile 0: 8 gate rows, tile 1: their 8 up rows -> 8 output columns
      const int tok = threadIdx.x >> 3, col = threadIdx.x & 7;
      if (threadIdx.x < 128 && tok < M && n0 / 2 + col < N / 2) {
        float g = 0.0f, u = 0.0f;
#pragma unroll
        for (int w = 0; w < SK_WARPS; ++w) {
          g += red[(w * TILES + 0) * 128 + tok * 8 + col];
          u += red[(w * TILES + (TILES - 1)) * 128 + tok * 8 + col];
        }
        g = __bfloat162float(__float2bfloat16_rn(g));
        u = __bfloat162float(__float2bfloat16_rn(u));
        out[tok * ldo + n0 / 2 + col] = from_float<OT>((g / (1.0f + expf(-g))) * u);
      }
    } else {
      for (int e = threadIdx.x; e < TILES * 128; e += SK_THREADS) {
        const int t = e >> 7, tok = (e & 127) >> 3, col = e & 7;
        if (tok < M && n0 + t * 8 + col < N) {
          float s = 0.0f;
#pragma unroll
          for (int w = 0; w < SK_WARPS; ++w) s += red[(w * TILES + t) * 128 + tok * 8 + col];
          out[tok * ldo + n0 + t * 8 + col] = from_float<OT>(s);
        }
      }
    }
    __syncthreads();                                       // red is reused by the next tile
  }
}

template <int MR, int TILES, int UN, bool NORM, bool SWIGLU, typename NW, typename OT = __nv_bfloat16>
static int launch_skinny(const void* x, const void* delta, void* x_out, const void* norm_w, float eps, const void* W,
                         void* out, int M, int N, int K, long long ldx, long long ldw, long long ldo,
                         cudaStream_t s) {
  const int smem = MR * (K + 8) * 2 + SK_WARPS * TILES * 128 * 4;
  static int smem_set = 0;                                 // per instance
  if (smem > 227 * 1024) return PIH_ERR_UNSUPPORTED;
  if (smem > 48 * 1024 && smem_set < smem) {
    cudaError_t e = cudaFuncSetAttribute(skinny_gemm_kernel<MR, TILES, UN, NORM, SWIGLU, NW, OT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    smem_set = smem;
  }
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  const int ntiles = (N + 8 * TILES - 1) / (8 * TILES);
  const int grid = ntiles < 2 * sms ? ntiles : 2 * sms;
  launch_kernel(skinny_gemm_kernel<MR, TILES, UN, NORM, SWIGLU, NW, OT>, dim3(grid), dim3(SK_THREADS), smem, s, 
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(delta),
      static_cast<__nv_bfloat16*>(x_out), static_cast<const NW*>(norm_w), eps,
      static_cast<const __nv_bfloat16*>(W), static_cast<OT*>(out), M, N, K, ldx, ldw, ldo);
  PIH_LAUNCH_CHECK();
  return 0;
}

template <int MR, bool NORM, typename NW>
static int dispatch_skinny(int tiles, bool swiglu, const void* x, const void* delta, void* x_out, const void* norm_w,
                           float eps, const void* W, void* out, int M, int N, int K, long long ldx, long long ldw,
                           long long ldo, cudaStream_t s) {
  if (swiglu)
    return launch_skinny<MR, 2, SK_UN, NORM, true, NW>(x, delta, x_out, norm_w, eps, W, out, M, N, K, ldx, ldw, ldo, s);
  if (tiles == 2)
    return launch_skinny<MR, 2, SK_UN, NORM, false, NW>(x, delta, x_out, norm_w, eps, W, out, M, N, K, ldx, ldw, ldo, s);
  // a long k with 8-row tiles: twice the loads in flight per warp, so that a block's life is one or two round
  // trips to memory instead of three (1024 x 3072: 5.6 -> 4.7 us; 1024 x 2048: 3.7 -> 3.4 us inside a step).
  // Pairs of blocks in a cluster that split k and add through distributed shared memory were measured too:
  // no faster than one block per tile (5.5 and 4.1 us).
  if (K > 32 * SK_WARPS * SK_UN)
    return launch_skinny<MR, 1, 2 * SK_UN, NORM, false, NW>(x, delta, x_out, norm_w, eps, W, out, M, N, K, ldx, ldw, ldo, s);
  return launch_skinny<MR, 1, SK_UN, NORM, false, NW>(x, delta, x_out, norm_w, eps, W, out, M, N, K, ldx, ldw, ldo, s);
}

}  // namespace pih

using namespace pih;

// bf16 only.  M <= 16 rows; K a multiple of 32; x rows, W rows and out rows 16-byte aligned.
//   delta      nullable: the rows are round(x + delta), as the fused add of a pre-norm block; the sums are also
//              written to x_out (a buffer other than x: CTAs read x while one of them writes)
//   norm_w     nullable: RMSNorm (weight dtype norm_dtype, eps) of the rows before the product
//   swiglu     W rows come in blocks of 16 = 8 gate rows + their 8 up rows; out is [M, N / 2]
// Returns PIH_ERR_UNSUPPORTED for shapes it does not take (the caller uses the separate kernels).
extern "C" int pih_gemm_skinny(const void* x, const void* delta, void* x_out, int norm_dtype, const void* norm_w,
                               float eps, const void* W, void* out, int M, int N, int K, long long ldx,
                               long long ldw, long long ldo, int swiglu, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 16 || K <= 0 || K % 32 || ldx % 8 || ldw % 8 || (swiglu && N % 16) ||
      (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(W) & 15) ||
      (reinterpret_cast<uintptr_t>(norm_w) & 15) ||
      (delta != nullptr && ((reinterpret_cast<uintptr_t>(delta) & 15) || x_out == nullptr || x_out == x)))
    return PIH_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // 16 weight rows per tile when that still gives every SM a tile, else 8
  const int tiles = (swiglu || N >= 148 * 16) ? 2 : 1;
  const bool sw = swiglu != 0;
#define PIH_SKINNY(MR, NORM, NW) \
  dispatch_skinny<MR, NORM, NW>(tiles, sw, x, delta, x_out, norm_w, eps, W, out, M, N, K, ldx, ldw, ldo, s)
  if (norm_w == nullptr) return M <= 8 ? PIH_SKINNY(8, false, float) : PIH_SKINNY(16, false, float);
  if (norm_dtype == PIH_F32) return M <= 8 ? PIH_SKINNY(8, true, float) : PIH_SKINNY(16, true, float);
  if (norm_dtype == PIH_BF16) return M <= 8 ? PIH_SKINNY(8, true, __nv_bfloat16) : PIH_SKINNY(16, true, __nv_bfloat16);
#undef PIH_SKINNY
  return PIH_ERR_BAD_ARGUMENT;
}

// The same product with 32-bit output and nothing fused: out[M, N] (float) = x[M, K] . W[N, K]^T, for the LM
// head of a decode step (the reference gives the head an fp32 output, src/backend/cuda/gemm_plan.cpp:111-113).
extern "C" int pih_gemm_skinny_f32out(const void* x, const void* W, void* out, int M, int N, int K, long long ldx,
                                      long long ldw, long long ldo, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 16 || K <= 0 || K % 32 || ldx % 8 || ldw % 8 || (reinterpret_cast<uintptr_t>(x) & 15) ||
      (reinterpret_cast<uintptr_t>(W) & 15))
    return PIH_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool wide = N >= 148 * 16;
#define PIH_SKINNY_F32(MR, TILES, UN) \
  launch_skinny<MR, TILES, UN, false, false, float, float>(x, nullptr, nullptr, nullptr, 0.0f, W, out, M, N, K, ldx, ldw, ldo, s)
  if (wide) return M <= 8 ? PIH_SKINNY_F32(8, 2, SK_UN) : PIH_SKINNY_F32(16, 2, SK_UN);
  if (K > 32 * SK_WARPS * SK_UN) return M <= 8 ? PIH_SKINNY_F32(8, 1, 2 * SK_UN) : PIH_SKINNY_F32(16, 1, 2 * SK_UN);
  return M <= 8 ? PIH_SKINNY_F32(8, 1, SK_UN) : PIH_SKINNY_F32(16, 1, SK_UN);
#undef PIH_SKINNY_F32
}
