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
