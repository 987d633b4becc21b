// Per-head RMSNorm and rotate-half rotation of one q or k head that a warp holds as EPL contiguous elements per
// lane (head_dim = 32 * EPL): the arithmetic and the rounding places of the reference's separate kernels — one
// rounding after the norm, one after the rotation (kernels/cuda/qwen_bf16_primitives.cu:285-347).  Shared by the
// q/k kernel (elementwise.cu) and by the decode attention kernel that does this work itself (attention_mma.cu),
// so that both give the same bits.
#pragma once
#include "common.cuh"

namespace pih {

// v: the lane's elements (32-bit); w: the lane's norm weights (nullptr: no norm); cs: (cos, sin) of the lane's
// pairs, pair index (lane & 15) * EPL + j (nullptr: no rotation).  The rotation partner of a lane is lane ^ 16.
// Every lane of the warp must call it.  On return v holds the values as they are stored (rounded to T).
template <typename T, typename W, int EPL>
__device__ __forceinline__ void head_norm_rotate(float (&v)[EPL], const W* w, float eps, const float2* cs, int lane) {
  constexpr int D = 32 * EPL;
  if (w != nullptr) {
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) ss += v[j] * v[j];
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / static_cast<float>(D) + eps);
#pragma unroll
    for (int j = 0; j < EPL; ++j) v[j] = round_to<T>((v[j] * scale) * to_float<W>(w[j]));
  }
  if (cs != nullptr) {
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const float other = __shfl_xor_sync(0xffffffffu, v[j], 16);
      const float c = cs[j].x, sn = cs[j].y;
      const float r = lane < 16 ? v[j] * c - other * sn : v[j] * c + other * sn;
      v[j] = round_to<T>(r);
    }
  }
}

}  // namespace pih
