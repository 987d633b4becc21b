// Products with few rows (decode: 1..16 tokens): out[M,N] = act[M,K] . W[N,K]^T, bound by reading W once.
//
// The reference pads every decode step to 4096 rows and calls cuBLASLt for each of q, k, v, o, gate, up and
// down (plugins/model-qwen3/nvidia_qwen3_bf16_engine.cpp:391-392; src/backend/cuda/gemm_plan.cpp:192-197),
// with RMSNorm, residual add and SiLU-mul as kernels of their own between them
// (kernels/cuda/qwen_bf16_primitives.cu:264-324).  Here one kernel streams the weight rows once and does
// the small work around the product itself.  A decode step is a chain of such kernels, each a few
// microseconds long; a kernel cannot start its arithmetic before the kernel before it has finished (it needs
// that kernel's output rows), so what decides the step's speed is how little remains to be done after that
// moment.  The kernel is shaped for that:
//
//   one block per SM   of 8 warps, at most half of an SM's registers and as much shared memory as the block's share
//              of the weights needs: the block of the NEXT kernel of the step fits beside it;
//   weights in shared memory, before the wait   no kernel writes weights, so the block's share of them is copied
//              into shared memory BEFORE griddepcontrol.wait, that is while the kernel before this one is still
//              running: a stage per unit of 8 or 16 weight rows, a bulk copy (cp.async.bulk, completion on the
//              stage's mbarrier) per row, issued by a lane each.  A block's whole share (50 to 100 KB at the sizes
//              of a 0.6B model) is in flight at once; longer jobs (the output head) walk over their units through a
//              ring of stages.  What was measured on the way: the SM's copy engine spends about 40 ns on a copy
//              whatever its size, so copies have to be whole rows (2 to 6 KB), not parts of rows; rows are padded by
//              64 bytes in shared memory, or the eight rows that a warp reads at once share their banks and reading
//              the weights back — 64 KB through a 128-byte-a-cycle port, on every block's path after the wait —
//              takes twice as long; and loading the weights into registers instead (no read-back at all) stalls on
//              the number of loads an SM can have in flight, long before its share is on its way.
//   the signal         when a block has issued its last weight load it executes griddepcontrol.launch_dependents:
//              once every block has done so, the next kernel's blocks become resident beside these and start their
//              own loads — memory has work at every moment;
//   prologue           after the wait: the token rows arrive by one bulk copy into shared memory; optional RMSNorm in
//              place, a warp per row (every block does this for itself from the few KB of rows: cheaper than a
//              kernel of its own and a round trip); optional residual add first (h <- round(h + delta), written
//              back once) when the product before this one has not added it in its own epilogue;
//   product            mma.sync m16n8k16; a thread's 16 bytes of a weight row per 32-wide k block are both halves of
//              its operand for two MMAs (the k order inside a block is permuted the same way for both operands,
//              which a dot product does not notice).  With at most 8 tokens the unit's 16 WEIGHT rows are the 16-row
//              operand and the tokens the 8-column one (no lane is wasted on tokens that do not exist); with 9 to 16
//              the tokens are the 16-row operand.  The eight warps split a unit's k: warp w takes k blocks w, w + 8, ...;
//   epilogue           the warps' partial sums meet in shared memory and are added in warp order; then store, or
//              out = round(round(sum) + residual) (the residual add that follows an output projection), or SwiGLU
//              when the unit's 16 rows are 8 gate rows followed by their 8 up rows:
//              out = round(silu(round(g)) * round(u))  (rounding places of the separate kernels).
//
// A row's result does not depend on the other rows of the batch (up to 8 rows, and 9 to 16 rows, are two
// arrangements of the same sums).  The one wait on an mbarrier is bounded and reports kWaitTimedOut.
#include "ptx.cuh"

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

// global -> this block's shared memory, `bytes` a multiple of 16, both addresses 16-byte aligned; completion is
// counted on the mbarrier
__device__ __forceinline__ void bulk_copy(void* smem_dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::
                   "r"(smem_u32(smem_dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

constexpr int SK_WARPS = 8;
constexpr int SK_THREADS = SK_WARPS * 32;
constexpr int SK_MAX_STAGES = 6;
constexpr int SK_HEAD_BYTES = 128;                           // the barriers

struct SkinnyParams {
  const __nv_bfloat16* x;
  const __nv_bfloat16* delta;
  __nv_bfloat16* x_out;
  const void* norm_w;
  const __nv_bfloat16* W;
  void* out;
  const __nv_bfloat16* residual;                 // nullable: out = round(round(product) + residual), rows of ldo elements
  float eps;
  int M, N, K;
  long long ldx, ldw, ldo;
  int stages;                                    // of the ring of units
  uint32_t* error;
};

// MR: rows of the token operand kept in shared memory (8 or 16).  T8: 8-row groups of weight rows in a unit
// (1 or 2; SwiGLU: 2, the 8 gate rows and their 8 up rows).
template <int MR, int T8, bool NORM, bool SWIGLU, typename NW, typename OT>
__global__ void __launch_bounds__(SK_THREADS, 2) skinny_gemm_kernel(const SkinnyParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int ROWS = 8 * T8;
  constexpr int NS = MR == 8 ? 1 : T8;                     // accumulator tiles of a unit
  constexpr int RED = NS * 128;                            // partial sums of a warp
  constexpr bool PAIRED = SWIGLU && MR == 8;               // gate and up of an output lie in one lane's accumulator
  const int K = p.K, N = p.N, M = p.M;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, q = lane & 3;
  uint64_t* xbar = reinterpret_cast<uint64_t*>(smem);                                    // the token rows have landed
  uint64_t* full = xbar + 1;                                                               // [stages] a unit has landed
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem + SK_HEAD_BYTES);            // [MR][K], as in memory
  float* red = reinterpret_cast<float*>(xs + MR * K);                                     // [2][SK_WARPS][RED]
  const NW* nws = reinterpret_cast<const NW*>(red + 2 * SK_WARPS * RED);                  // [K] the norm's weights
  const int row_bytes = K * 2 + 64;                        // a stage's rows alternate between the halves of the bank window
  const int stage_bytes = ROWS * row_bytes;
  unsigned char* ring = smem + ((SK_HEAD_BYTES + MR * K * 2 + 2 * SK_WARPS * RED * 4 + (NORM ? K * static_cast<int>(sizeof(NW)) : 0) + 127) / 128) * 128;
  const int S = p.stages;

  const int KB = K / 32;                                   // k blocks
  const int nunits = (N + ROWS - 1) / ROWS;
  const int my_units = blockIdx.x < nunits ? (nunits - 1 - blockIdx.x) / gridDim.x + 1 : 0;
  if (threadIdx.x == 0) {
    mbar_init(xbar, 1);
    for (int s = 0; s < S; ++s) mbar_init(&full[s], 1);
    mbar_init_fence();
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // the copy engine sees the barriers as initialised
  }
  __syncthreads();

  // ---- the weights: the block's unit `u` goes to stage u % S; its rows are copied by all eight warps, row r by
  // lane r / 8 of warp r % 8 (the copy engine takes requests from several warps faster than a row after the other
  // from one)
  auto issue_unit = [&](int u) {
    const int unit = blockIdx.x + u * gridDim.x;
    const int rows = min(ROWS, N - unit * ROWS);
    uint64_t* bar = &full[u % S];
    if (threadIdx.x == 0) mbar_expect_tx(bar, static_cast<uint32_t>(rows * K * 2));
    const int r = warp + SK_WARPS * lane;
    if (lane < T8 && r < rows)
      bulk_copy(ring + (u % S) * stage_bytes + r * row_bytes, p.W + (static_cast<long long>(unit) * ROWS + r) * p.ldw,
                static_cast<uint32_t>(K * 2), bar);
  };
  for (int u = 0; u < min(S, my_units); ++u) issue_unit(u);
  // the block's last weight copy is on its way (all of a block's warps get here at about the same time)
  if (threadIdx.x == 0 && my_units <= S) launch_dependents();

  const int chunks16 = K / 8;                              // 16-byte chunks of a token row
  // rows beyond the batch are zero (nothing to wait for)
  for (int row = M + warp; row < MR; row += SK_WARPS) {
    __nv_bfloat16* xrow = xs + row * K;
    for (int c = lane; c < chunks16; c += 32) *reinterpret_cast<uint4*>(xrow + c * 8) = make_uint4(0, 0, 0, 0);
  }
  wait_for_prior_kernels();
  if (my_units == 0) return;

  // ---- the epilogue's thread map: thread e < 128 (PAIRED: < 64) owns one output of a unit — or one of each 8-row
  // group — given by a lane and an accumulator register of the MMA; its residual value is asked for a unit early
  const int el = PAIRED ? threadIdx.x >> 1 : threadIdx.x >> 2;      // the lane whose accumulator it reads
  const int er = PAIRED ? threadIdx.x & 1 : threadIdx.x & 3;        // ... and which register of it
  const int egid = el >> 2, eq = el & 3;
  // MR == 8: register r of lane (gid, q) is weight row gid + 8 (r / 2) of the unit for token 2 q + (r & 1);
  // MR == 16: token gid + 8 (r / 2) at column 2 q + (r & 1) of each 8-row group
  const int etok = MR == 8 ? 2 * eq + (er & 1) : egid + 8 * (er >> 1);
  const int ecol = MR == 8 ? egid + 8 * (er >> 1) : 2 * eq + (er & 1);
  const bool eactive = threadIdx.x < (PAIRED ? 64 : 128) && etok < M;
  float res_next = 0.0f;
  auto load_residual = [&](int unit_index) {
    if (SWIGLU || p.residual == nullptr || !eactive || unit_index >= my_units) return;
    const int col = (blockIdx.x + unit_index * gridDim.x) * ROWS + ecol;
    if (col < N && (MR == 16 || T8 == 2 || ecol < 8)) res_next = __bfloat162float(p.residual[etok * p.ldo + col]);
  };
  load_residual(0);

  // ---- the token rows
  const NW* norm_w = static_cast<const NW*>(p.norm_w);
  constexpr int NWV = 8 * sizeof(NW) / 16;                 // 16-byte loads per 8 norm weights
  if (p.delta == nullptr) {
    // one bulk copy for all of them.  Every block of the kernel asks for the same few KB at the same moment, so
    // this trip to the L2 is the slowest part of a block's life.
    if (warp == 0) {
      const uint32_t norm_bytes = NORM ? static_cast<uint32_t>(K * sizeof(NW)) : 0u;
      if (lane == 0) mbar_expect_tx(xbar, static_cast<uint32_t>(M * K * 2) + norm_bytes);
      __syncwarp();
      if (p.ldx == K) {
        if (lane == 0) bulk_copy(xs, p.x, static_cast<uint32_t>(M * K * 2), xbar);
      } else if (lane < M) {
        bulk_copy(xs + lane * K, p.x + lane * p.ldx, static_cast<uint32_t>(K * 2), xbar);
      }
      if (NORM && lane == 31) bulk_copy(const_cast<NW*>(nws), p.norm_w, norm_bytes, xbar);   // the norm's weights beside them
    }
    mbar_wait(xbar, 0, p.error);
    if (NORM) {
      // warp w norms rows w, w + 8 in place: a few hundred dependent instructions of one warp, on every block's
      // path.  Two chunks of a lane at a time (the weights of the product hold most of the registers), their
      // squares in sums of their own.
      for (int row = warp; row < M; row += SK_WARPS) {
        __nv_bfloat16* xrow = xs + row * K;
        float s2[2] = {0.0f, 0.0f};
        for (int c0 = lane; c0 < chunks16; c0 += 64) {
          uint4 v[2];
#pragma unroll
          for (int j = 0; j < 2; ++j)
            v[j] = c0 + 32 * j < chunks16 ? *reinterpret_cast<const uint4*>(xrow + (c0 + 32 * j) * 8) : make_uint4(0, 0, 0, 0);
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const __nv_bfloat162* ve = reinterpret_cast<const __nv_bfloat162*>(&v[j]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = __bfloat1622float2(ve[e]);
              s2[j] = fmaf(f.x, f.x, s2[j]);
              s2[j] = fmaf(f.y, f.y, s2[j]);
            }
          }
        }
        const float ss = warp_sum(s2[0] + s2[1]);
        const float scale = 1.0f / sqrtf(ss / static_cast<float>(K) + p.eps);
        for (int c0 = lane; c0 < chunks16; c0 += 64) {
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int c = c0 + 32 * j;
            if (c >= chunks16) continue;
            uint4 v = *reinterpret_cast<const uint4*>(xrow + c * 8);
            uint4 wq[NWV];
#pragma unroll
            for (int u = 0; u < NWV; ++u) wq[u] = *(reinterpret_cast<const uint4*>(nws + c * 8) + u);
            const NW* we = reinterpret_cast<const NW*>(wq);
            __nv_bfloat16* ve = reinterpret_cast<__nv_bfloat16*>(&v);
#pragma unroll
            for (int e = 0; e < 8; ++e)
              ve[e] = __float2bfloat16_rn((__bfloat162float(ve[e]) * scale) * to_float<NW>(we[e]));
            *reinterpret_cast<uint4*>(xrow + c * 8) = v;
          }
        }
      }
    }
  } else {
    // with a residual to add first (the product before this one did not add it itself): warp w prepares token
    // rows w, w + 8 through registers.  A lane takes chunks lane, lane + 32, ..., four at a time with their loads
    // issued together; the sum is rounded and kept (one block writes it out), its squares are summed on the way,
    // and the normed row replaces it in shared memory.
    for (int row = warp; row < M; row += SK_WARPS) {
      __nv_bfloat16* xrow = xs + row * K;
      float ss = 0.0f;
      for (int c0 = 0; c0 < chunks16; c0 += 128) {
        uint4 v[4], d[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int c = c0 + lane + 32 * j;
          v[j] = d[j] = make_uint4(0, 0, 0, 0);
          if (c < chunks16) {
            v[j] = *reinterpret_cast<const uint4*>(p.x + row * p.ldx + c * 8);
            d[j] = *reinterpret_cast<const uint4*>(p.delta + row * p.ldx + c * 8);
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int c = c0 + lane + 32 * j;
          if (c >= chunks16) continue;
          __nv_bfloat16* ve = reinterpret_cast<__nv_bfloat16*>(&v[j]);
          const __nv_bfloat16* de = reinterpret_cast<const __nv_bfloat16*>(&d[j]);
#pragma unroll
          for (int e = 0; e < 8; ++e) ve[e] = __float2bfloat16_rn(__bfloat162float(ve[e]) + __bfloat162float(de[e]));
          // the sum goes to a buffer of its own: other blocks are still reading x
          if (blockIdx.x == 0) *reinterpret_cast<uint4*>(p.x_out + row * p.ldx + c * 8) = v[j];
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
        const float scale = 1.0f / sqrtf(ss / static_cast<float>(K) + p.eps);
        for (int c = lane; c < chunks16; c += 32) {
          uint4 wq[NWV];
#pragma unroll
          for (int u = 0; u < NWV; ++u) wq[u] = ldg_nc16(reinterpret_cast<const uint4*>(norm_w + c * 8) + u);
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

  // ---- the product: unit after unit from its stage; warp w takes k blocks w, w + 8, ...; two chains of accumulators
  OT* out = static_cast<OT*>(p.out);
  const unsigned char* xa = reinterpret_cast<const unsigned char*>(xs) + gid * K * 2 + q * 16;   // token gid's row
  float acc[2][NS][4];
  auto zero_acc = [&]() {
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
      for (int t = 0; t < NS; ++t) acc[a][t][0] = acc[a][t][1] = acc[a][t][2] = acc[a][t][3] = 0.0f;
  };
  zero_acc();
  // the end of a unit: partial sums to shared memory, one barrier, the owners add them in warp order and store.
  // Two buffers in turn: a warp writes for the unit after next only after the barrier of the next unit, which
  // every thread reaches only when it has read this unit's sums.
  auto finish_unit = [&](int unit_index) {
    float* mine = red + ((unit_index & 1) * SK_WARPS + warp) * RED;
#pragma unroll
    for (int t = 0; t < NS; ++t)
      *reinterpret_cast<float4*>(mine + t * 128 + lane * 4) =
          make_float4(acc[0][t][0] + acc[1][t][0], acc[0][t][1] + acc[1][t][1], acc[0][t][2] + acc[1][t][2],
                      acc[0][t][3] + acc[1][t][3]);
    zero_acc();
    __syncthreads();
    const float res_now = res_next;
    load_residual(unit_index + 1);
    if (!eactive) return;
    const float* all = red + (unit_index & 1) * SK_WARPS * RED;
    const int n0 = (blockIdx.x + unit_index * gridDim.x) * ROWS;
    if (SWIGLU) {
      // the unit's rows 0..7 are gate rows, rows 8..15 their up rows
      constexpr int UP = MR == 8 ? 2 : 128;                // where the up row's sum lies from the gate row's
      float g = 0.0f, u = 0.0f;
#pragma unroll
      for (int w = 0; w < SK_WARPS; ++w) {
        g += all[w * RED + el * 4 + er];
        u += all[w * RED + el * 4 + er + UP];
      }
      const int col = n0 / 2 + (MR == 8 ? egid : ecol);
      if (col < N / 2) {
        g = __bfloat162float(__float2bfloat16_rn(g));
        u = __bfloat162float(__float2bfloat16_rn(u));
        out[etok * p.ldo + col] = from_float<OT>((g / (1.0f + expf(-g))) * u);
      }
    } else {
#pragma unroll
      for (int t = 0; t < NS; ++t) {
        const int col = n0 + (MR == 8 ? ecol : 8 * t + ecol);
        if (col >= N || (MR == 8 && T8 == 1 && ecol >= 8)) continue;
        float sum = 0.0f;
#pragma unroll
        for (int w = 0; w < SK_WARPS; ++w) sum += all[w * RED + t * 128 + el * 4 + er];
        // (a residual never comes with two 8-row groups of 16 tokens: see the dispatch)
        if (p.residual != nullptr) sum = __bfloat162float(__float2bfloat16_rn(sum)) + res_now;
        out[etok * p.ldo + col] = from_float<OT>(sum);
      }
    }
  };

  for (int u = 0; u < my_units; ++u) {
    mbar_wait(&full[u % S], (u / S) & 1, p.error);
    const unsigned char* wb = ring + (u % S) * stage_bytes + gid * row_bytes + q * 16;
    for (int kb0 = warp; kb0 < KB; kb0 += 2 * SK_WARPS) {
#pragma unroll
      for (int a = 0; a < 2; ++a) {
        const int kb = kb0 + a * SK_WARPS;
        if (kb >= KB) break;
        const uint4 xlo = *reinterpret_cast<const uint4*>(xa + kb * 64);
        if constexpr (MR == 8) {
          const uint4 wlo = *reinterpret_cast<const uint4*>(wb + kb * 64);
          uint4 whi = make_uint4(0, 0, 0, 0);
          if (T8 == 2) whi = *reinterpret_cast<const uint4*>(wb + 8 * row_bytes + kb * 64);
          mma16816(acc[a][0], wlo.x, whi.x, wlo.y, whi.y, xlo.x, xlo.y);
          mma16816(acc[a][0], wlo.z, whi.z, wlo.w, whi.w, xlo.z, xlo.w);
        } else {
          const uint4 xhi = *reinterpret_cast<const uint4*>(xa + 8 * K * 2 + kb * 64);
#pragma unroll
          for (int t = 0; t < T8; ++t) {
            const uint4 w = *reinterpret_cast<const uint4*>(wb + t * 8 * row_bytes + kb * 64);
            mma16816(acc[a][t], xlo.x, xhi.x, xlo.y, xhi.y, w.x, w.y);
            mma16816(acc[a][t], xlo.z, xhi.z, xlo.w, xhi.w, w.z, w.w);
          }
        }
      }
    }
    finish_unit(u);                                        // (its barrier: every warp has read the stage)
    // the stage is free: the unit S places on comes into it
    if (u + S < my_units) {
      issue_unit(u + S);
      if (threadIdx.x == 0 && u + S == my_units - 1) launch_dependents();
    }
  }
}

template <int MR, int T8, bool NORM, bool SWIGLU, typename NW, typename OT = __nv_bfloat16>
static int launch_skinny(SkinnyParams p, cudaStream_t s) {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  constexpr int RED = (MR == 8 ? 1 : T8) * 128;
  const int nunits = (p.N + 8 * T8 - 1) / (8 * T8);
  const int grid = nunits < sms ? nunits : sms;
  const int per_block = (nunits + grid - 1) / grid;        // units of the busiest block
  const int head = ((SK_HEAD_BYTES + MR * p.K * 2 + 2 * SK_WARPS * RED * 4 + (NORM ? p.K * static_cast<int>(sizeof(NW)) : 0) + 127) / 128) * 128;
  const int stage = 8 * T8 * (p.K * 2 + 64);
  // A stage for every unit of the block when that stays within about half of an SM's shared memory (the next kernel's
  // block then fits beside this one); a block with many units to walk over (the output head) runs for long and takes
  // what keeps an SM's share of the memory bandwidth in flight instead.
  int stages = per_block < SK_MAX_STAGES ? per_block : SK_MAX_STAGES;
  const int budget = (per_block > 4 ? 200 : 160) * 1024;
  while (stages > 1 && head + stages * stage > budget) --stages;
  const int smem = head + stages * stage;
  if (smem > 227 * 1024) return PIH_ERR_UNSUPPORTED;
  p.stages = stages;
  static int smem_set = -1;                                // per instance
  if (smem_set < 0) {
    // Every kernel of a decode step asks for the same split of an SM's memory between L1 and shared memory (all
    // of it shared): blocks of two kernels whose preferences differ cannot be resident on an SM at the same time,
    // and the next kernel's blocks would wait for the SM to drain instead of starting beside this one's.
    cudaError_t e = cudaFuncSetAttribute(skinny_gemm_kernel<MR, T8, NORM, SWIGLU, NW, OT>,
                                         cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return static_cast<int>(e);
    smem_set = 0;
  }
  if (smem > 48 * 1024 && smem_set < smem) {
    cudaError_t e = cudaFuncSetAttribute(skinny_gemm_kernel<MR, T8, NORM, SWIGLU, NW, OT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    smem_set = smem;
  }
  launch_kernel(skinny_gemm_kernel<MR, T8, NORM, SWIGLU, NW, OT>, dim3(grid), dim3(SK_THREADS), smem, s, p);
  PIH_LAUNCH_CHECK();
  return 0;
}

template <int MR, bool NORM, typename NW>
static int dispatch_skinny(bool swiglu, const SkinnyParams& p, cudaStream_t s) {
  if (swiglu) return launch_skinny<MR, 2, NORM, true, NW>(p, s);
  // units of 16 weight rows when that still gives every SM one (for few tokens they cost no more MMAs than 8 rows)
  if (MR == 8 && p.N >= 148 * 16) return launch_skinny<MR, 2, NORM, false, NW>(p, s);
  return launch_skinny<MR, 1, NORM, false, NW>(p, s);
}

// ---- the same product for a LONG job: many weight rows per SM (the output head: a vocabulary of rows) -----------
//
// The kernel above is made for a block that owns a few units and lives for a few microseconds.  The output head
// gives every SM a megabyte of weights; what counts there is only how many bytes an SM keeps in flight, and a
// stage ring with a block-wide meeting per unit does not keep enough.  Here nothing is staged and no warp ever
// waits for another: a warp owns 8-row granules of W (granule g of warp w of block b: w * blocks + b + g * warps),
// loads a granule's rows straight into registers in the MMA's operand layout — a lane's 16 bytes of a row per 32-wide
// k block are the 8-column operand of two MMAs, as above — eight k blocks at a time into one of two register sets,
// the next set's loads issued before this set's MMAs.  Sixteen warps an SM with up to 8 KB each on the way cover the
// memory's latency.  The tokens (up to 16 rows, padded rows as above) lie in shared memory and are the 16-row
// operand.  A warp's sums are complete in its own accumulators: it stores them, 32 bytes a token.
constexpr int SH_WARPS = 8;
constexpr int SH_CHUNK = 8;                                  // k blocks of a register set

template <int MR, typename OT>
__global__ void __launch_bounds__(SH_WARPS * 32, 2) skinny_stream_kernel(const SkinnyParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int K = p.K, N = p.N, M = p.M;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, q = lane & 3;
  const int row_bytes = K * 2 + 64;
  const int KB = K / 32;
  const int chunks = (KB + SH_CHUNK - 1) / SH_CHUNK;        // register sets of a granule
  const int granules = (N + 7) / 8;
  const int warps = gridDim.x * SH_WARPS;
  const int gw = warp * gridDim.x + blockIdx.x;              // (the granules left over go to different SMs)
  const int my_granules = gw < granules ? (granules - 1 - gw) / warps + 1 : 0;
  const int items = my_granules * chunks;

  // the next set to load: granule and chunk of it
  int lg = gw, lc = 0;
  auto load_set = [&](uint4 (&set)[SH_CHUNK]) {
    const int row = min(lg * 8 + gid, N - 1);                // (rows beyond the last are loaded twice and not stored)
    const unsigned char* src = reinterpret_cast<const unsigned char*>(p.W + static_cast<long long>(row) * p.ldw) +
                               q * 16 + lc * (SH_CHUNK * 64);
#pragma unroll
    for (int j = 0; j < SH_CHUNK; ++j)
      if (lc * SH_CHUNK + j < KB) set[j] = ldg_nc16(src + j * 64);
    if (++lc == chunks) lc = 0, lg += warps;
  };

  uint4 set_a[SH_CHUNK], set_b[SH_CHUNK];
  if (items > 0) load_set(set_a);                            // weights: nobody writes them, so before the wait
  wait_for_prior_kernels();
  launch_dependents();                                       // (what follows the head is small: it may wait beside it)

  // the token rows, padded so that the eight rows a warp reads at once lie in different banks; rows beyond M zero
  const int chunks16 = K / 8;
  for (int i = threadIdx.x; i < MR * chunks16; i += SH_WARPS * 32) {
    const int row = i / chunks16, c = i - row * chunks16;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < M) v = *reinterpret_cast<const uint4*>(p.x + row * p.ldx + c * 8);
    *reinterpret_cast<uint4*>(smem + row * row_bytes + c * 16) = v;
  }
  __syncthreads();

  OT* out = static_cast<OT*>(p.out);
  const unsigned char* xa = smem + gid * row_bytes + q * 16;
  float acc[2][4];
  int cg = gw, cc = 0;                                       // the set to use: granule and chunk of it
  auto use_set = [&](const uint4 (&set)[SH_CHUNK]) {
    if (cc == 0) {
#pragma unroll
      for (int a = 0; a < 2; ++a) acc[a][0] = acc[a][1] = acc[a][2] = acc[a][3] = 0.0f;
    }
#pragma unroll
    for (int j = 0; j < SH_CHUNK; ++j) {
      const int kb = cc * SH_CHUNK + j;
      if (kb < KB) {
        const uint4 xlo = *reinterpret_cast<const uint4*>(xa + kb * 64);
        uint4 xhi = make_uint4(0, 0, 0, 0);
        if (MR == 16) xhi = *reinterpret_cast<const uint4*>(xa + 8 * row_bytes + kb * 64);
        mma16816(acc[j & 1], xlo.x, xhi.x, xlo.y, xhi.y, set[j].x, set[j].y);
        mma16816(acc[j & 1], xlo.z, xhi.z, xlo.w, xhi.w, set[j].z, set[j].w);
      }
    }
    if (++cc == chunks) {
      // register r of lane (gid, q): token gid + 8 (r / 2), weight row 2 q + (r & 1) of the granule
      const int col = cg * 8 + 2 * q;
#pragma unroll
      for (int h = 0; h < MR / 8; ++h) {
        const int tok = gid + 8 * h;
        if (tok < M) {
          OT* o = out + tok * p.ldo + col;
          if (col < N) o[0] = from_float<OT>(acc[0][2 * h] + acc[1][2 * h]);
          if (col + 1 < N) o[1] = from_float<OT>(acc[0][2 * h + 1] + acc[1][2 * h + 1]);
        }
      }
      cc = 0, cg += warps;
    }
  };

  for (int i = 0; i < items; i += 2) {
    if (i + 1 < items) load_set(set_b);
    use_set(set_a);
    if (i + 2 < items) load_set(set_a);
    if (i + 1 < items) use_set(set_b);
  }
}

static int stream_sms() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  return sms;
}
// a job for the streaming kernel: every warp of a full grid (two blocks an SM) gets at least four granules
static bool stream_takes(const SkinnyParams& p) { return (p.N + 7) / 8 >= 4 * (2 * stream_sms()) * SH_WARPS; }

// Takes the job when every warp of its grid gets at least four granules; returns PIH_ERR_UNSUPPORTED otherwise.
template <int MR, typename OT>
static int launch_stream(const SkinnyParams& p, cudaStream_t s) {
  const int sms = stream_sms();
  const int smem = MR * (p.K * 2 + 64);
  const int per_sm = smem <= 100 * 1024 ? 2 : 1;
  if (smem > 200 * 1024) return PIH_ERR_UNSUPPORTED;
  const int grid = sms * per_sm;
  if ((p.N + 7) / 8 < 4 * grid * SH_WARPS) return PIH_ERR_UNSUPPORTED;
  static int smem_set = 0;
  if (smem > 48 * 1024 && smem_set < smem) {
    cudaError_t e = cudaFuncSetAttribute(skinny_stream_kernel<MR, OT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    smem_set = smem;
  }
  launch_kernel(skinny_stream_kernel<MR, OT>, dim3(grid), dim3(SH_WARPS * 32), smem, s, p);
  PIH_LAUNCH_CHECK();
  return 0;
}

static bool skinny_takes(const void* x, const void* W, int M, int K, long long ldx, long long ldw) {
  return M <= 16 && K > 0 && K % 32 == 0 && ldx % 8 == 0 && ldw % 8 == 0 &&
         (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(W) & 15) == 0;
}

int g_skinny_rule = 1;

}  // namespace pih

using namespace pih;

// 1 (the default): pih_gemm_skinny declines the shapes for which the library's product is the faster way; 0: it takes
// every shape it can (for measurements of the kernel itself).  Returns the previous setting.
extern "C" int pih_set_skinny_rule(int on) {
  const int before = pih::g_skinny_rule;
  pih::g_skinny_rule = on ? 1 : 0;
  return before;
}

// bf16 only.  M <= 16 rows; K a multiple of 32; x rows, W rows and out rows 16-byte aligned.
//   delta      nullable: the rows are round(x + delta), as the fused add of a pre-norm block; the sums are also
//              written to x_out (a buffer other than x: blocks read x while one of them writes)
//   norm_w     nullable: RMSNorm (weight dtype norm_dtype, eps) of the rows before the product
//   swiglu     W rows come in blocks of 16 = 8 gate rows + their 8 up rows; out is [M, N / 2]
//   residual   nullable (not with swiglu): out = round(round(x . W^T) + residual), the residual add that follows an
//              output projection, with its two roundings; rows of ldo elements; may not be `out` itself
//   error      the device's error word (a bounded wait that ran out is reported there)
// Returns PIH_ERR_UNSUPPORTED for shapes it does not take (the caller uses the separate kernels).
extern "C" int pih_gemm_skinny(const void* x, const void* delta, void* x_out, int norm_dtype, const void* norm_w,
                               float eps, const void* W, void* out, const void* residual, int M, int N, int K,
                               long long ldx, long long ldw, long long ldo, int swiglu, uint32_t* error, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (!skinny_takes(x, W, M, K, ldx, ldw) || (swiglu && (N % 16 || residual != nullptr)) ||
      (reinterpret_cast<uintptr_t>(norm_w) & 15) || residual == out || (norm_w != nullptr && K % 8) ||
      (delta != nullptr && ((reinterpret_cast<uintptr_t>(delta) & 15) || x_out == nullptr || x_out == x)))
    return PIH_ERR_UNSUPPORTED;
  // Where the library's product with the separate norm, SiLU-mul and add kernels is the faster way (measured at the
  // Qwen3-0.6B, 1.7B and 8B layer sizes, 8 and 16 rows, weights larger than L2 between calls), the caller is sent there:
  // up to 8 rows this kernel wins until a block's share of the weights passes what shared memory holds several times
  // (gate/up 24576 x 4096: 46 against 36 + 5 us) or the norm of rows of 4096 is repeated by every block (q/k/v 6144 x
  // 4096: 16.4 against 11.8 + 3); with 9 to 16 rows only at the smallest sizes (6144 x 1024: 7.2 against 5.8 + 5;
  // 12288 x 2048: 21.9 against 11.7 + 5; 6144 x 4096: 26.5 against 12.8 + 3).
  if (g_skinny_rule) {
    const long long weight_bytes = static_cast<long long>(N) * K * 2;
    const bool slower = M <= 8 ? (weight_bytes > (64ll << 20) || (norm_w != nullptr && K >= 4096))
                               : weight_bytes > (13ll << 20);
    if (slower) return PIH_ERR_UNSUPPORTED;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  SkinnyParams p = {};
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.delta = static_cast<const __nv_bfloat16*>(delta);
  p.x_out = static_cast<__nv_bfloat16*>(x_out);
  p.norm_w = norm_w;
  p.W = static_cast<const __nv_bfloat16*>(W);
  p.out = out;
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.eps = eps;
  p.M = M, p.N = N, p.K = K;
  p.ldx = ldx, p.ldw = ldw, p.ldo = ldo;
  p.error = error;
  const bool sw = swiglu != 0;
#define PIH_SKINNY(MR, NORM, NW) dispatch_skinny<MR, NORM, NW>(sw, p, s)
  if (norm_w == nullptr) return M <= 8 ? PIH_SKINNY(8, false, float) : PIH_SKINNY(16, false, float);
  if (norm_dtype == PIH_F32) return M <= 8 ? PIH_SKINNY(8, true, float) : PIH_SKINNY(16, true, float);
  if (norm_dtype == PIH_BF16) return M <= 8 ? PIH_SKINNY(8, true, __nv_bfloat16) : PIH_SKINNY(16, true, __nv_bfloat16);
#undef PIH_SKINNY
  return PIH_ERR_BAD_ARGUMENT;
}

// The same product with 32-bit output and nothing fused: out[M, N] (float) = x[M, K] . W[N, K]^T, for the LM
// head of a decode step (the reference gives the head an fp32 output, src/backend/cuda/gemm_plan.cpp:111-113).
extern "C" int pih_gemm_skinny_f32out(const void* x, const void* W, void* out, int M, int N, int K, long long ldx,
                                      long long ldw, long long ldo, uint32_t* error, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (!skinny_takes(x, W, M, K, ldx, ldw)) return PIH_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  SkinnyParams p = {};
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.W = static_cast<const __nv_bfloat16*>(W);
  p.out = out;
  p.M = M, p.N = N, p.K = K;
  p.ldx = ldx, p.ldw = ldw, p.ldo = ldo;
  p.error = error;
  // A vocabulary of rows: the kernel for long jobs, if the job is long enough for it and has at most 8 rows.  With 9 to
  // 16 rows the library's product is the faster one for such a job (151 936 weight rows, fp32 out, k = 1024 / 2048 /
  // 4096: 57 / 106 / 213 us against this kernel's 64 / 120 / 375; at 8 rows 56 / 104 / 210 against 54 / 99 / 202):
  // the caller is told to use it.
  if (stream_takes(p)) {
    if (M > 8) return PIH_ERR_UNSUPPORTED;
    const int rc = launch_stream<8, float>(p, s);
    if (rc != PIH_ERR_UNSUPPORTED) return rc;
  }
  if (M <= 8)
    return N >= 148 * 16 ? launch_skinny<8, 2, false, false, float, float>(p, s)
                         : launch_skinny<8, 1, false, false, float, float>(p, s);
  return launch_skinny<16, 1, false, false, float, float>(p, s);
}
