// The few-rows product as a device function: the body of skinny_gemm_kernel (gemm_skinny.cu) and of the stages of
// skinny_chain_kernel (gemm_chain.cu).  See gemm_skinny.cu for what it computes and how.
#pragma once
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
// CHAINED: the product is a stage of a chain inside one kernel (gemm_chain.cu): instead of waiting for the
// kernel before it, it waits at a barrier of the whole grid (`barrier`, after its first weight loads are in
// flight), reads the token rows past the L1 cache (other blocks wrote them in this kernel) and blocks without a
// tile skip the stage.  Returns false when the barrier gave up.
template <int MR, int TILES, int UN, bool NORM, bool SWIGLU, typename NW, typename OT, bool CHAINED, typename Barrier>
__device__ __forceinline__ bool skinny_gemm_body(unsigned char* smem_raw, const __nv_bfloat16* __restrict__ x,
                                                 const __nv_bfloat16* __restrict__ delta,
                                                 __nv_bfloat16* __restrict__ x_out, const NW* __restrict__ norm_w,
                                                 float eps, const __nv_bfloat16* __restrict__ W, OT* __restrict__ out,
                                                 int M, int N, int K, long long ldx, long long ldw, long long ldo,
                                                 Barrier barrier) {
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
  const bool has_tile = tile < ntiles;
  // neither the weight stream nor the norm weights wait for the prologue or for the kernel before this one
  // (no kernel writes weights): the first loads are in flight while that kernel's last blocks finish
  if (has_tile) issue(tile, warp);
  const int chunks = K / 8;                                // 16-byte chunks of a token row
  constexpr int NWV = 8 * sizeof(NW) / 16;                 // 16-byte loads per 8 norm weights
  uint4 wpre[4][NWV];                                      // norm weights of the lane's first four chunks
  if (NORM && has_tile) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = lane + 32 * j;
#pragma unroll
      for (int v = 0; v < NWV; ++v)
        wpre[j][v] = c < chunks ? ldg_nc16(reinterpret_cast<const uint4*>(norm_w + c * 8) + v) : make_uint4(0, 0, 0, 0);
    }
  }
  if (CHAINED) {
    if (!barrier()) return false;
    if (!has_tile) return true;
  } else {
    wait_for_prior_kernels();
  }
  auto load16 = [](const __nv_bfloat16* p) {
    return CHAINED ? __ldcg(reinterpret_cast<const uint4*>(p)) : *reinterpret_cast<const uint4*>(p);
  };

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
          v[j] = load16(x + row * ldx + c * 8);
          if (delta != nullptr) d[j] = load16(delta + row * ldx + c * 8);
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
  return true;
}

}  // namespace pih
