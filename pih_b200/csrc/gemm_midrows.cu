// Products with 17 to 64 rows (decode steps of that many requests): out[M,N] = act[M,K] . W[N,K]^T, bound by
// reading W once — if the token rows do not have to be read once per SM as well.
//
// The few-rows kernel (gemm_skinny.cu) keeps all token rows in every block's shared memory; 64 rows of 6144 do
// not fit, and 148 blocks fetching them all from the L2 would move more bytes than the weights are.  Here a
// CLUSTER of 2, 4 or 8 blocks shares a slice of the weight rows and splits k: block c of the cluster keeps only
// columns [c K/C, (c+1) K/C) of the token rows in its shared memory (64 rows x 1536 columns: 196 KB) and
// multiplies them with the same columns of the slice's weight rows; the partial sums of the cluster's blocks
// meet through distributed shared memory, each block adding up and storing a share of the slice's outputs in
// block order.  The reference pads such a step to 4096 rows and calls cuBLASLt
// (plugins/model-qwen3/nvidia_qwen3_bf16_engine.cpp:391-392); the library's own kernels for these shapes take
// 34 us a layer at the 1.7B sizes against 15 us of weight traffic.  This kernel is correct and not yet faster:
// 45 us for the same four products (its fixed costs — two cluster barriers, the sums through distributed shared
// memory, token columns fetched after the wait — are about 6 us a product), so the engine keeps the library's
// products for these row counts unless told otherwise (CudaOps.midrows_product).
//
//   weights    straight from global memory into registers in the MMA's operand layout, as in the output head's
//              kernel (a lane's 16 bytes of a row per 32-wide k block are the 8-column operand of two
//              mma.sync.m16n8k16): a warp owns UNITS of 16 weight rows (two 8-row operands side by side, so that a
//              token fragment read from shared memory serves both) and loads four k blocks of a unit at a time
//              into one of two register sets, the next set's loads issued before this set's MMAs.  The first set
//              is asked for before griddepcontrol.wait: no kernel writes weights.
//   tokens     this block's columns of the up to 64 rows, padded rows as in gemm_skinny.cu; they are the 16-row
//              operand, MT tiles of 16 rows.
//   epilogue   partial sums (the raw accumulators, 16 bytes a lane) into the block's shared memory over the token
//              columns, which are no longer needed; cluster barrier; unit u of the slice is finished by block
//              u % C: sum over the blocks in rank order, then store, or out = round(round(sum) + residual), or
//              SwiGLU when a unit is 8 gate rows followed by their 8 up rows (rounding places of the separate
//              kernels); a second cluster barrier keeps every block's memory alive until all have read.
//
// No mbarrier, no spin: the block and cluster barriers are hardware barriers that every thread reaches.
#include "ptx.cuh"

namespace pih {

__device__ __forceinline__ void mid_mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 mid_ldg_nc16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t mid_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void mid_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// 16 bytes from the shared memory of block `rank` of the cluster, at the address that `local` has in this block's
__device__ __forceinline__ float4 mid_load_from_block(const float4* local, uint32_t rank) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(local));
  uint32_t remote;
  float4 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(a), "r"(rank));
  asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(remote)
               : "memory");
  return v;
}

constexpr int MID_WARPS = 8;
constexpr int MID_THREADS = MID_WARPS * 32;
constexpr int MID_CHUNK = 8;                              // k blocks of a register set

struct MidParams {
  const __nv_bfloat16* x;
  const __nv_bfloat16* W;
  __nv_bfloat16* out;
  const __nv_bfloat16* residual;                 // nullable: out = round(round(product) + residual), rows of ldo elements
  int M, N, K;
  long long ldx, ldw, ldo;
  int cluster;                                   // blocks of a cluster = parts of k
  int kb_per_block;                              // 32-wide k blocks of a part
  int units_per_cluster;                         // 16-row units of weight rows of a cluster's slice
  int parked_offset;                             // bytes: where a warp keeps the sums of its units but the last
};

// MT: 16-row tiles of token rows (2..4).
template <int MT, bool SWIGLU>
__global__ void __launch_bounds__(MID_THREADS, 1) midrows_gemm_kernel(const MidParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int K = p.K, N = p.N, M = p.M;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, q = lane & 3;
  const int C = p.cluster;
  const int rank = static_cast<int>(mid_cluster_rank());
  const int slice = blockIdx.x / C;
  const int KB = K / 32;
  const int kb0 = min(KB, rank * p.kb_per_block), kb1 = min(KB, kb0 + p.kb_per_block);
  const int nkb = kb1 - kb0;                               // this block's k blocks (0: it only takes part in the sums)
  const int units = (N + 15) / 16;
  const int u0 = slice * p.units_per_cluster;
  const int nunits = max(0, min(units, u0 + p.units_per_cluster) - u0);
  const int row_bytes = p.kb_per_block * 64 + 64;          // padded: the eight rows a warp reads at once lie in different banks
  const int chunks = (nkb + MID_CHUNK - 1) / MID_CHUNK;
  const int my_units = warp < nunits ? (nunits - 1 - warp) / MID_WARPS + 1 : 0;
  const int items = my_units * chunks;

  // the next set to load: unit (of this warp) and chunk of it
  int lu = warp, lc = 0;
  auto load_set = [&](uint4 (&set)[2][MID_CHUNK]) {
    const int n0 = (u0 + lu) * 16;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = min(n0 + 8 * h + gid, N - 1);        // (rows beyond the last are loaded twice and not stored)
      const unsigned char* src = reinterpret_cast<const unsigned char*>(p.W + static_cast<long long>(row) * p.ldw) +
                                 (kb0 + lc * MID_CHUNK) * 64 + q * 16;
#pragma unroll
      for (int j = 0; j < MID_CHUNK; ++j)
        if (lc * MID_CHUNK + j < nkb) set[h][j] = mid_ldg_nc16(src + j * 64);
    }
    if (++lc == chunks) lc = 0, lu += MID_WARPS;
  };

  uint4 set_a[2][MID_CHUNK], set_b[2][MID_CHUNK];
  // weights: nobody writes them, so two sets are asked for before the wait (a warp's whole share, in the usual case)
  if (items > 0) load_set(set_a);
  if (items > 1) load_set(set_b);
  wait_for_prior_kernels();
  launch_dependents();

  // this block's columns of the token rows; rows beyond M zero
  {
    const int per_row = nkb * 4;                           // 16-byte pieces
    const __nv_bfloat16* x0 = p.x + kb0 * 32;
    for (int i = threadIdx.x; i < 16 * MT * per_row; i += MID_THREADS) {
      const int row = i / per_row, c = i - row * per_row;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (row < M) v = *reinterpret_cast<const uint4*>(x0 + row * p.ldx + c * 8);
      *reinterpret_cast<uint4*>(smem + row * row_bytes + c * 16) = v;
    }
  }
  __syncthreads();

  const unsigned char* xa = smem + gid * row_bytes + q * 16;
  float acc[2][MT][4];
  float4* part = reinterpret_cast<float4*>(smem);          // [unit of the slice][half][tile][lane], over the token columns
  int cu = warp, cc = 0;                                   // the set to use: unit (of this warp) and chunk of it
  bool wrote = false;
  auto use_set = [&](const uint4 (&set)[2][MID_CHUNK]) {
    if (cc == 0) {
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int t = 0; t < MT; ++t) acc[h][t][0] = acc[h][t][1] = acc[h][t][2] = acc[h][t][3] = 0.0f;
    }
#pragma unroll
    for (int j = 0; j < MID_CHUNK; ++j) {
      const int kb = cc * MID_CHUNK + j;
      if (kb < nkb) {
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          const uint4 xlo = *reinterpret_cast<const uint4*>(xa + 16 * t * row_bytes + kb * 64);
          const uint4 xhi = *reinterpret_cast<const uint4*>(xa + (16 * t + 8) * row_bytes + kb * 64);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            mid_mma16816(acc[h][t], xlo.x, xhi.x, xlo.y, xhi.y, set[h][j].x, set[h][j].y);
            mid_mma16816(acc[h][t], xlo.z, xhi.z, xlo.w, xhi.w, set[h][j].z, set[h][j].w);
          }
        }
      }
    }
    if (++cc == chunks) {
      cc = 0;
      // (kept in registers until every warp has finished with the token columns: see below)
      wrote = true;
    }
  };

  // A warp has at most a few units; the sums of a finished unit have to wait in registers for the barrier after
  // which the token columns may be overwritten, so a warp with more than one unit parks them in a part of shared
  // memory of its own behind the token columns.
  float4* parked = reinterpret_cast<float4*>(smem + p.parked_offset) + warp * (2 * MT * 32);
  int parked_units = 0;
  for (int i = 0; i < items; i += 2) {
    if (i > 0 && i + 1 < items) load_set(set_b);
    use_set(set_a);
    if (wrote) {
      wrote = false;
      if (cu + MID_WARPS < nunits) {                       // not this warp's last unit: park it
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int t = 0; t < MT; ++t)
            parked[(parked_units * MID_WARPS * 2 * MT + h * MT + t) * 32 + lane] =
                make_float4(acc[h][t][0], acc[h][t][1], acc[h][t][2], acc[h][t][3]);
        ++parked_units;
        cu += MID_WARPS;
      }
    }
    if (i + 2 < items) load_set(set_a);
    if (i + 1 < items) {
      use_set(set_b);
      if (wrote) {
        wrote = false;
        if (cu + MID_WARPS < nunits) {
#pragma unroll
          for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int t = 0; t < MT; ++t)
              parked[(parked_units * MID_WARPS * 2 * MT + h * MT + t) * 32 + lane] =
                  make_float4(acc[h][t][0], acc[h][t][1], acc[h][t][2], acc[h][t][3]);
          ++parked_units;
          cu += MID_WARPS;
        }
      }
    }
  }
  __syncthreads();                                         // every warp has read the token columns for the last time
  // the partial sums of the slice's units, unit by unit
  for (int k = 0; k < my_units; ++k) {
    const int u = warp + k * MID_WARPS;
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int t = 0; t < MT; ++t) {
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);    // (a block without k blocks adds nothing)
        if (nkb != 0) {
          if (k == my_units - 1) v = make_float4(acc[h][t][0], acc[h][t][1], acc[h][t][2], acc[h][t][3]);
          else v = parked[(k * MID_WARPS * 2 * MT + h * MT + t) * 32 + lane];
        }
        part[((u * 2 + h) * MT + t) * 32 + lane] = v;
      }
  }
  mid_cluster_sync();                                      // every block's partial sums are in place

  // unit u of the slice is finished by block u % C: a warp per (unit, tile) adds the blocks' sums in rank order,
  // all of their loads through distributed shared memory in flight at once
  const int owned = nunits > rank ? (nunits - 1 - rank) / C + 1 : 0;
  for (int task = warp; task < owned * MT; task += MID_WARPS) {
    const int u = rank + (task / MT) * C, t = task % MT;
    float4 v[2][8];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < C) v[h][r] = mid_load_from_block(&part[((u * 2 + h) * MT + t) * 32 + lane], static_cast<uint32_t>(r));
    float4 s[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      s[h] = v[h][0];
#pragma unroll
      for (int r = 1; r < 8; ++r)
        if (r < C) s[h].x += v[h][r].x, s[h].y += v[h][r].y, s[h].z += v[h][r].z, s[h].w += v[h][r].w;
    }
    // register r of lane (gid, q) of tile t: token 16 t + gid + 8 (r / 2), weight row 2 q + (r & 1) of the 8-row half
    const int n0 = (u0 + u) * 16;
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {                       // the two token rows of the lane
      const int tok = 16 * t + gid + 8 * hr;
      if (tok >= M) continue;
      if (SWIGLU) {
        const int col = n0 / 2 + 2 * q;
        const float g0 = hr ? s[0].z : s[0].x, g1 = hr ? s[0].w : s[0].y;
        const float v0 = hr ? s[1].z : s[1].x, v1 = hr ? s[1].w : s[1].y;
        const float gg[2] = {__bfloat162float(__float2bfloat16_rn(g0)), __bfloat162float(__float2bfloat16_rn(g1))};
        const float uu[2] = {__bfloat162float(__float2bfloat16_rn(v0)), __bfloat162float(__float2bfloat16_rn(v1))};
#pragma unroll
        for (int e = 0; e < 2; ++e)
          if (col + e < N / 2)
            p.out[tok * p.ldo + col + e] = __float2bfloat16_rn((gg[e] / (1.0f + expf(-gg[e]))) * uu[e]);
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int col = n0 + 8 * h + 2 * q;
          float o[2] = {hr ? s[h].z : s[h].x, hr ? s[h].w : s[h].y};
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            if (col + e >= N) continue;
            if (p.residual != nullptr)
              o[e] = __bfloat162float(__float2bfloat16_rn(o[e])) + __bfloat162float(p.residual[tok * p.ldo + col + e]);
            p.out[tok * p.ldo + col + e] = __float2bfloat16_rn(o[e]);
          }
        }
      }
    }
  }
  mid_cluster_sync();                                      // every block has read: all may go
}

template <int MT, bool SWIGLU>
static int launch_midrows(MidParams p, cudaStream_t s) {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  const int KB = p.K / 32;
  const int units = (p.N + 15) / 16;
  static bool attribute_set = false;
  if (!attribute_set) {
    cudaError_t e = cudaFuncSetAttribute(midrows_gemm_kernel<MT, SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
    attribute_set = true;
  }
  // How many clusters of 2, 4 and 8 blocks the device runs at once: a cluster lies within one group of SMs, so the
  // groups' remainders stay empty (148 SMs hold 32 clusters of 4, not 37), and a grid of more clusters than that
  // runs in two waves.  Asked once per size, with the most shared memory a block may take.
  static int resident[4] = {0, 0, 0, 0};                   // [log2 of the cluster size]
  auto clusters_at_once = [&](int c, int log2c) {
    if (resident[log2c] == 0) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(sms / c * c);
      cfg.blockDim = dim3(MID_THREADS);
      cfg.dynamicSmemBytes = 220 * 1024;
      cudaLaunchAttribute attr[1] = {};
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = c, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr, cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, midrows_gemm_kernel<MT, SWIGLU>, &cfg) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = sms / c * 3 / 4;                               // a guess on the safe side
      }
      resident[log2c] = n < sms / c ? n : sms / c;
    }
    return resident[log2c];
  };
  // The smallest cluster whose parts of the token rows fit a block's shared memory and that leaves every block
  // about a warp's worth of units or more (fewer blocks of a cluster = fewer partial sums to add).
  int chosen = 0, smem = 0, clusters_max = 0;
  for (int c = 2, log2c = 1; c <= 8; c *= 2, ++log2c) {
    const int kbs = (KB + c - 1) / c;
    int clusters = clusters_at_once(c, log2c);
    int upc = (units + clusters - 1) / clusters;
    const int x_bytes = 16 * MT * (kbs * 64 + 64);
    if (upc > MID_WARPS && x_bytes + ((upc + MID_WARPS - 1) / MID_WARPS - 1) * MID_WARPS * 2 * MT * 32 * 16 > 220 * 1024) {
      // no room to park a warp's second unit beside the token columns: a unit a warp, in more clusters than run at once
      upc = MID_WARPS;
      clusters = (units + upc - 1) / upc;
    }
    const int rounds = (upc + MID_WARPS - 1) / MID_WARPS;
    const int parked = rounds > 1 ? (rounds - 1) * MID_WARPS * 2 * MT * 32 * 16 : 0;
    const int part_bytes = upc * 2 * MT * 32 * 16;
    const int front = x_bytes > part_bytes ? x_bytes : part_bytes;
    const int need = front + parked;
    if (need > 220 * 1024) continue;
    chosen = c, smem = need, clusters_max = clusters;
    p.parked_offset = front;
    if (upc >= 6 || c == 8) break;
  }
  if (chosen == 0) return PIH_ERR_UNSUPPORTED;
  p.cluster = chosen;
  p.kb_per_block = (KB + chosen - 1) / chosen;
  p.units_per_cluster = (units + clusters_max - 1) / clusters_max;
  const int clusters = (units + p.units_per_cluster - 1) / p.units_per_cluster;
  launch_kernel_clustered(midrows_gemm_kernel<MT, SWIGLU>, dim3(clusters * chosen), dim3(MID_THREADS), smem, s,
                          static_cast<unsigned>(chosen), p);
  PIH_LAUNCH_CHECK();
  return 0;
}

}  // namespace pih

using namespace pih;

// bf16 only.  17 <= M <= 64 rows; K a multiple of 32; x rows, W rows and out rows 16-byte aligned.
//   swiglu     W rows come in blocks of 16 = 8 gate rows + their 8 up rows; out is [M, N / 2]
//   residual   nullable (not with swiglu): out = round(round(x . W^T) + residual); rows of ldo elements; not `out`
// Returns PIH_ERR_UNSUPPORTED for shapes it does not take (the caller uses the library product).
extern "C" int pih_gemm_midrows(const void* x, const void* W, void* out, const void* residual, int M, int N, int K,
                                long long ldx, long long ldw, long long ldo, int swiglu, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M <= 16 || M > 64 || K <= 0 || K % 32 || ldx % 8 || ldw % 8 || (reinterpret_cast<uintptr_t>(x) & 15) ||
      (reinterpret_cast<uintptr_t>(W) & 15) || (swiglu && (N % 16 || residual != nullptr)) || residual == out)
    return PIH_ERR_UNSUPPORTED;
  MidParams p = {};
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.W = static_cast<const __nv_bfloat16*>(W);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.M = M, p.N = N, p.K = K;
  p.ldx = ldx, p.ldw = ldw, p.ldo = ldo;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int mt = (M + 15) / 16;
  if (swiglu) return mt == 2 ? launch_midrows<2, true>(p, s) : mt == 3 ? launch_midrows<3, true>(p, s) : launch_midrows<4, true>(p, s);
  return mt == 2 ? launch_midrows<2, false>(p, s) : mt == 3 ? launch_midrows<3, false>(p, s) : launch_midrows<4, false>(p, s);
}
