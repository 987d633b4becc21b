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
#include "gemm_skinny_body.cuh"

namespace pih {

struct NoBarrier {
  __device__ bool operator()() const { return true; }
};

template <int MR, int TILES, int UN, bool NORM, bool SWIGLU, typename NW, typename OT>
__global__ void __launch_bounds__(SK_THREADS)
skinny_gemm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                   __nv_bfloat16* __restrict__ x_out, const NW* __restrict__ norm_w, float eps,
                   const __nv_bfloat16* __restrict__ W, OT* __restrict__ out, int M, int N, int K,
                   long long ldx, long long ldw, long long ldo) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  skinny_gemm_body<MR, TILES, UN, NORM, SWIGLU, NW, OT, false>(smem_raw, x, delta, x_out, norm_w, eps, W, out, M, N, K,
                                                              ldx, ldw, ldo, NoBarrier());
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
