// Shared device helpers of the pih_b200 kernel pack (sm_100a).
//
// Storage types: float (the true 32-bit path) and __nv_bfloat16 (serving).
// All arithmetic inside an op is fp32; a value is rounded once where it is
// stored, with round-to-nearest-even, as the reference's store_bf16 does
// (kernels/cuda/qwen_bf16_primitives.cu:16-24).
//
// Errors found on the device (a token id outside the table, a row that maps
// to no page, a non-finite value where none may be) never trap: the kernel
// records the first code in one device word and carries on with a harmless
// value, and the host reads the word with the step's results — the
// reference's error_flag discipline (qwen_bf16_primitives.cu:89-94).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace pih {

enum ErrorCode : uint32_t {
  kOk = 0,
  kTokenOutOfVocabulary = 1,
  kRowWithoutPage = 2,
  kNonFiniteLogit = 3,
  kBadPosition = 4,
  kAttentionDenominator = 5,
  kWaitTimedOut = 6,
};

// A step may be padded to a larger shape: a row of padding carries this cache slot (nothing is written for it) and
// request -1; a request of padding has no rows.  Kernels leave both alone without reporting anything.
constexpr int kPaddingSlot = -2;

__device__ __forceinline__ void publish_error(uint32_t* flag, uint32_t code) {
  if (flag != nullptr) atomicCAS(flag, 0u, code);
}

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// round a 32-bit value to the storage type and back
template <typename T> __device__ __forceinline__ float round_to(float v) {
  return to_float<T>(from_float<T>(v));
}

// silu(g) * u in 32-bit.  The 32-bit stream uses expf and a true division, as the reference's kernel does
// (kernels/cuda/qwen_bf16_primitives.cu:274-283); the bf16 stream uses the special-function unit's exp2 and
// reciprocal, whose two-ulp error in 32-bit is a five-hundredth of a bf16 rounding step.
template <typename T> __device__ __forceinline__ float silu_times(float g, float u);
template <> __device__ __forceinline__ float silu_times<float>(float g, float u) { return (g / (1.0f + expf(-g))) * u; }
template <> __device__ __forceinline__ float silu_times<__nv_bfloat16>(float g, float u) {
  return __fdividef(g, 1.0f + __expf(-g)) * u;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The
// order of additions depends only on blockDim, never on other rows or blocks.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < warps ? scratch[lane] : 0.0f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Programmatic dependent launch.  Kernels of the pack are launched with programmatic stream serialisation:
// the next kernel's blocks may become resident as soon as every block of the kernel before it has exited or
// has executed launch_dependents(), before that kernel's writes have been flushed; wait_for_prior_kernels()
// then blocks until every earlier kernel has completed and its writes are visible.  Every kernel launched
// through launch_kernel() executes the wait in its blocks before their first read of anything an earlier
// kernel may have written and before their first write to global memory (only loads of what no kernel writes
// — weights, the cache of earlier steps, the step's batch arrays — may come before it), so completion of a
// kernel implies completion of all kernels before it.  The kernels of a decode step signal their dependents
// when their last load from memory has been issued, and are shaped so that the next kernel's block fits on
// the SM beside theirs (one block per SM, half its registers, about 100 KB of its shared memory): the next
// kernel's first loads are in flight while this one computes and stores.  Both instructions do nothing in a
// kernel launched without the attribute.  The reference launches every kernel with full serialisation
// (kernels/cuda/qwen_bf16_primitives.cu, all launches).
__device__ __forceinline__ void wait_for_prior_kernels() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// 1: kernels are launched with programmatic stream serialisation; 0: plain launches.  Set by pih_set_dependent_launch.
extern int g_dependent_launch;

// cluster_x > 1: thread-block clusters of that many blocks along x (grid.x must be a multiple of it)
template <typename... P, typename... A>
inline void launch_kernel_clustered(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    unsigned cluster_x, A&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2] = {};
  unsigned n = 0;
  if (g_dependent_launch) {
    attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_x > 1) {
    attrs[n].id = cudaLaunchAttributeClusterDimension;
    attrs[n].val.clusterDim.x = cluster_x;
    attrs[n].val.clusterDim.y = 1;
    attrs[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = n;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);   // the caller reads cudaGetLastError()
}

template <typename... P, typename... A>
inline void launch_kernel(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A&&... args) {
  launch_kernel_clustered(kernel, grid, block, smem, stream, 1u, static_cast<A&&>(args)...);
}

}  // namespace pih

// dtype codes of the C entry points
#define PIH_F32 0
#define PIH_BF16 1

// C entry points return 0, a cudaError_t (> 0) from the launch, or one of these
#define PIH_ERR_BAD_ARGUMENT (-1)
#define PIH_ERR_UNSUPPORTED (-2)

#define PIH_LAUNCH_CHECK()                                  \
  do {                                                      \
    cudaError_t e_ = cudaGetLastError();                    \
    if (e_ != cudaSuccess) return static_cast<int>(e_);     \
  } while (0)
