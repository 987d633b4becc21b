// A chain of few-rows products in ONE persistent kernel: stage s + 1 reads what stage s wrote, with a barrier
// of the whole grid between them.
//
// A decode step is bound by reading the weights once, but as separate kernels each product pays a launch, the
// latency of its first loads and its last blocks' tail: four products of a layer took 20 us for 31 MB, which
// HBM delivers in 5.  Here every block issues the first weight loads of the NEXT stage (weights depend on
// nothing) and only then waits at the barrier, so the memory system never drains between stages.  The stages
// are the products of gemm_skinny.cu with their fused prologues and epilogues (gemm_skinny_body.cuh); the
// chain that the engine runs is the tail of a pre-norm block:
//     o = attn . Wo^T;   h' = h + o;   act = SwiGLU(RMSNorm(h') . Wgu^T);   y = act . Wd^T
// The reference runs these as seven library products and three kernels
// (plugins/model-qwen3/qwen3_bf16_execution_schedule.cpp:40-64).
//
// Measured (Qwen3-0.6B shapes, batch 8, inside the decode step's CUDA graph): the chain is SLOWER than its three
// kernels launched with programmatic stream serialisation — 1.342 against 1.197 ms a step, 5 us a layer.  A
// barrier of 296 blocks (arrivals on one word, release seen by polling through L2) costs about two
// microseconds, which is what a kernel boundary costs there.  The engine therefore leaves it off
// (CudaOps.chain_block_tail); it stays as a tested option.
//
// The barrier counts arrivals in a device word and releases by a generation word; every wait is bounded
// (about two seconds), after which the block records kWaitTimedOut and returns.  The kernel is launched
// cooperatively, so the driver refuses it unless all its blocks can be resident together.  The two words live
// in the library: launches that may overlap on the GPU (several streams) must not use this entry point.
#include "gemm_skinny_body.cuh"

namespace pih {

constexpr long long kBarrierWaitCycles = 4000000000LL;   // about two seconds of SM clock

__device__ unsigned int g_chain_arrived = 0;
__device__ unsigned int g_chain_generation = 0;

__device__ __forceinline__ unsigned int load_acquire(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct GridBarrier {
  uint32_t* error;
  __device__ bool operator()() const {
    __shared__ int s_ok;
    __syncthreads();                                       // this block's writes of the stage are done
    if (threadIdx.x == 0) {
      int ok = 1;
      const unsigned int generation = load_acquire(&g_chain_generation);
      __threadfence();                                     // the block's writes before its arrival
      if (atomicAdd(&g_chain_arrived, 1u) == gridDim.x - 1) {
        g_chain_arrived = 0;                               // the last block resets the count, then releases
        __threadfence();
        atomicAdd(&g_chain_generation, 1u);
      } else {
        const long long t0 = clock64();
        while (load_acquire(&g_chain_generation) == generation) {
          if (clock64() - t0 > kBarrierWaitCycles) {
            publish_error(error, kWaitTimedOut);
            ok = 0;
            break;
          }
        }
      }
      __threadfence();
      s_ok = ok;
    }
    __syncthreads();
    return s_ok != 0;
  }
};

// one stage: out = [SwiGLU] ([RMSNorm] (x [+ delta])) . W^T
struct ChainStage {
  const __nv_bfloat16* x;
  const __nv_bfloat16* delta;        // nullable
  __nv_bfloat16* x_out;              // x + delta, when delta is given
  const void* norm_w;                // nullable
  float eps;
  const __nv_bfloat16* W;
  __nv_bfloat16* out;
  int N, K;
  long long ldx, ldw, ldo;
  int kind;                          // 0 plain, 1 norm, 2 norm + SwiGLU
  int variant;                       // 0: 8-row tiles, 4 k blocks in flight; 1: 8-row tiles, 8 in flight; 2: 16-row tiles
};

struct ChainArgs {
  ChainStage stage[3];
  int M;
  uint32_t* error;
};

struct NoWait {
  __device__ bool operator()() const { return true; }
};

// a stage without norm: 8- or 16-row weight tiles, 4 or 8 k blocks in flight, by the host's choice
template <int MR, typename NW, typename Barrier>
__device__ __forceinline__ bool plain_stage(unsigned char* smem, const ChainStage& st, int M, Barrier barrier) {
  if (st.variant == 2)
    return skinny_gemm_body<MR, 2, SK_UN, false, false, NW, __nv_bfloat16, true>(
        smem, st.x, nullptr, nullptr, static_cast<const NW*>(nullptr), 0.0f, st.W, st.out, M, st.N, st.K, st.ldx, st.ldw,
        st.ldo, barrier);
  if (st.variant == 1)
    return skinny_gemm_body<MR, 1, 2 * SK_UN, false, false, NW, __nv_bfloat16, true>(
        smem, st.x, nullptr, nullptr, static_cast<const NW*>(nullptr), 0.0f, st.W, st.out, M, st.N, st.K, st.ldx, st.ldw,
        st.ldo, barrier);
  return skinny_gemm_body<MR, 1, SK_UN, false, false, NW, __nv_bfloat16, true>(
      smem, st.x, nullptr, nullptr, static_cast<const NW*>(nullptr), 0.0f, st.W, st.out, M, st.N, st.K, st.ldx, st.ldw,
      st.ldo, barrier);
}

// plain product; add + norm + product + SwiGLU; plain product
template <int MR, typename NW>
__global__ void __launch_bounds__(SK_THREADS, 2) skinny_chain_kernel(const __grid_constant__ ChainArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  wait_for_prior_kernels();
  const GridBarrier barrier{a.error};
  if (!plain_stage<MR, NW>(smem_raw, a.stage[0], a.M, NoWait())) return;
  {
    const ChainStage& st = a.stage[1];
    if (!skinny_gemm_body<MR, 2, SK_UN, true, true, NW, __nv_bfloat16, true>(
            smem_raw, st.x, st.delta, st.x_out, static_cast<const NW*>(st.norm_w), st.eps, st.W, st.out, a.M, st.N, st.K,
            st.ldx, st.ldw, st.ldo, barrier))
      return;
  }
  plain_stage<MR, NW>(smem_raw, a.stage[2], a.M, barrier);
}

}  // namespace pih

using namespace pih;

// The tail of a pre-norm block for at most 16 rows (bf16), as one kernel:
//   o = attn [M, Ka] . w_o [H, Ka]^T;  h_out = round(h + o);  act = SwiGLU(RMSNorm(h_out; norm_w, eps) . w_gu [2 I, H]^T)
//   y = act . w_down [H, I]^T
// w_gu rows come in blocks of 16 = 8 gate rows + their 8 up rows.  o, h_out, act and y are buffers of the
// caller ([M, H], [M, H], [M, I], [M, H], contiguous).  norm_dtype: PIH_BF16 or PIH_F32.  Returns
// PIH_ERR_UNSUPPORTED for shapes it does not take (the caller runs the separate kernels).
extern "C" int pih_block_tail_chain(const void* attn, long long ld_attn, int Ka, const void* w_o, long long ld_wo,
                                    const void* h, void* o, void* h_out, int norm_dtype, const void* norm_w, float eps,
                                    const void* w_gu, long long ld_wgu, int I, void* act, const void* w_down,
                                    long long ld_wd, void* y, int M, int H, uint32_t* error, void* stream) {
  if (M <= 0) return 0;
  const auto misaligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
  if (M > 16 || H <= 0 || I <= 0 || Ka <= 0 || H % 32 || Ka % 32 || I % 32 || I % 8 || H % 8 || ld_attn % 8 ||
      ld_wo % 8 || ld_wgu % 8 || ld_wd % 8 || misaligned(attn) || misaligned(w_o) || misaligned(h) || misaligned(o) ||
      misaligned(h_out) || misaligned(norm_w) || misaligned(w_gu) || misaligned(act) || misaligned(w_down) ||
      misaligned(y) || norm_w == nullptr)
    return PIH_ERR_UNSUPPORTED;
  if (norm_dtype != PIH_BF16 && norm_dtype != PIH_F32) return PIH_ERR_BAD_ARGUMENT;
  ChainArgs a = {};
  a.M = M;
  a.error = error;
  const auto plain_variant = [](int N, int K) { return N >= 148 * 16 ? 2 : (K > 32 * SK_WARPS * SK_UN ? 1 : 0); };
  a.stage[0] = {static_cast<const __nv_bfloat16*>(attn), nullptr, nullptr, nullptr, 0.0f,
                static_cast<const __nv_bfloat16*>(w_o), static_cast<__nv_bfloat16*>(o), H, Ka, ld_attn, ld_wo, H, 0,
                plain_variant(H, Ka)};
  a.stage[1] = {static_cast<const __nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(o),
                static_cast<__nv_bfloat16*>(h_out), norm_w, eps, static_cast<const __nv_bfloat16*>(w_gu),
                static_cast<__nv_bfloat16*>(act), 2 * I, H, H, ld_wgu, I, 2, 2};
  a.stage[2] = {static_cast<const __nv_bfloat16*>(act), nullptr, nullptr, nullptr, 0.0f,
                static_cast<const __nv_bfloat16*>(w_down), static_cast<__nv_bfloat16*>(y), H, I, I, ld_wd, H, 0,
                plain_variant(H, I)};
  const int MR = M <= 8 ? 8 : 16;
  int kmax = Ka > H ? Ka : H;
  if (I > kmax) kmax = I;
  const int smem = MR * (kmax + 8) * 2 + SK_WARPS * 2 * 128 * 4;
  if (2 * (smem + 1024) > 227 * 1024) return PIH_ERR_UNSUPPORTED;      // two blocks per SM
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * sms);                             // lowered below if fewer blocks fit an SM
  cfg.blockDim = dim3(SK_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr = {};
  attr.id = cudaLaunchAttributeCooperative;                // all blocks resident together, or the launch fails
  attr.val.cooperative = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
#define PIH_CHAIN(MRV, NW)                                                                                   \
  do {                                                                                                       \
    static int smem_set = 0, resident = 0;                                                                   \
    if (smem_set < smem) {                                                                                   \
      if (smem > 48 * 1024) {                                                                                \
        cudaError_t e = cudaFuncSetAttribute(skinny_chain_kernel<MRV, NW>,                                   \
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);             \
        if (e != cudaSuccess) return static_cast<int>(e);                                                    \
      }                                                                                                      \
      smem_set = smem;                                                                                       \
      /* blocks of this kernel that fit an SM with this much shared memory: the grid must be resident whole */ \
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, skinny_chain_kernel<MRV, NW>, SK_THREADS,  \
                                                        smem) != cudaSuccess)                                \
        resident = 0;                                                                                        \
    }                                                                                                        \
    if (resident < 1) return PIH_ERR_UNSUPPORTED;                                                            \
    cfg.gridDim = dim3((resident < 2 ? resident : 2) * sms);                                                 \
    cudaLaunchKernelEx(&cfg, skinny_chain_kernel<MRV, NW>, a);                                               \
  } while (0)
  if (norm_dtype == PIH_BF16) {
    if (MR == 8) PIH_CHAIN(8, __nv_bfloat16);
    else PIH_CHAIN(16, __nv_bfloat16);
  } else {
    if (MR == 8) PIH_CHAIN(8, float);
    else PIH_CHAIN(16, float);
  }
#undef PIH_CHAIN
  PIH_LAUNCH_CHECK();
  return 0;
}

// After a barrier that gave up (kWaitTimedOut), the barrier's words may be left out of their resting state:
// this puts them back.  Call it with no chain kernel running.
extern "C" int pih_block_tail_chain_reset() {
  const unsigned int zero = 0;
  cudaError_t e = cudaMemcpyToSymbol(g_chain_arrived, &zero, sizeof(zero));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_chain_generation, &zero, sizeof(zero));
  return static_cast<int>(e);
}
