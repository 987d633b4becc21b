// Products with few rows (decode: 1..16 tokens): out[M,N] = act[M,K] . W[N,K]^T, bound by reading W once.
//
// The reference pads every decode step to 4096 rows and calls cuBLASLt for each of q, k, v, o, gate, up and
// down (plugins/model-qwen3/nvidia_qwen3_bf16_engine.cpp:391-392; src/backend/cuda/gemm_plan.cpp:192-197),
// with RMSNorm, residual add and SiLU-mul as kernels of their own between them
// (kernels/cuda/qwen_bf16_primitives.cu:264-324).  Here one kernel streams the weight rows once and does
// the small work around the product itself.  A decode step is a chain of such kernels, each a few
// microseconds long, so what decides its speed is whether the stream of weights from memory keeps running
// across the boundaries between them.  The kernel is shaped for that:
//
//   one block per SM   of 8 consumer warps and one producer warp, at most half of an SM's registers and about
//              100 KB of its shared memory: the block of the NEXT kernel of the step fits beside it;
//   weight ring        the producer's elected lane copies weight rows into a ring of stages in shared memory
//              with bulk copies (cp.async.bulk, completion on an mbarrier per stage); a stage is TN weight rows
//              (8 or 16) x 512 columns; the block walks over tiles blockIdx.x, + gridDim.x, ...;
//   before the wait    no kernel writes weights, so the ring is filled BEFORE griddepcontrol.wait, that is while
//              the kernel before this one is still running — its last blocks compute while this kernel's first
//              megabytes are already in flight;
//   the signal         when the producer has issued the block's last copy it executes
//              griddepcontrol.launch_dependents: once every block has done so, the next kernel's blocks become
//              resident beside these and start filling their rings — the memory pipe has work at every moment;
//   prologue           after the wait: optional residual add (h <- round(h + delta), written back once) and RMSNorm
//              of the M rows into shared memory, a warp per row, recomputed by every block from the few KB of rows
//              (cheaper than a kernel of its own and a round trip);
//   product            mma.sync m16n8k16 with the TOKENS as the 16-row operand and 8 weight rows as the 8-column
//              operand; a thread reads 16 contiguous bytes of a row per 32-wide k block from the stage (the k order
//              inside a block is permuted the same way for both operands, which a dot product does not notice);
//              the eight warps take every eighth k block of a stage, and their partial sums are added in a fixed
//              order when a tile's last stage is done;
//   epilogue           store, or SwiGLU when the tile's 16 weight rows are 8 gate rows followed by their 8 up rows:
//              out = round(silu(round(g)) * round(u))  (rounding places of the separate kernels).
//
// A row's result does not depend on the other rows of the batch.  Every wait on an mbarrier is bounded; a wait
// that runs out records kWaitTimedOut, the block stops waiting (its output is then meaningless, the host sees the
// error word), waits — bounded again — for the copies it still has in flight, and returns.
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
// counted on the mbarrier.  The weights are read once: they are marked to leave L2 first.
__device__ __forceinline__ void bulk_copy(void* smem_dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;\n" ::
          "r"(smem_u32(smem_dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void bulk_copy_keep(void* smem_dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::
                   "r"(smem_u32(smem_dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ uint64_t evict_first_policy() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(p));
  return p;
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 256;\n" ::: "memory"); }

constexpr int SK_WARPS = 8;
constexpr int SK_THREADS = SK_WARPS * 32;
constexpr int SK_KR_MAX = 1024;                  // most columns of a part: a row of a stage is ONE bulk copy of up to 2 KB
constexpr int SK_MAX_DEPTH = 4;
constexpr int SK_X_PAD = 0;                      // token rows lie as in memory: one bulk copy brings them all
constexpr int SK_HEAD_BYTES = 512;               // barriers

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
  int ksplit;                                    // 1, 2, 4 or 8 warps share the k of a sub-tile
  int kr;                                        // columns of a part, a multiple of 32
  int depth;                                     // stages of a warp's ring
  int groups;                                    // warp groups of a block that have work (rings exist for these only)
  uint32_t* error;
  int trigger;                                   // debug: 0 none, 1 after the last issue, 2 at the top
  unsigned long long* stamps;                    // debug: [16] per block
  int stamp_mask;
};
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define STAMP(k) do { if (p.stamps != nullptr && lane == 0 && warp == 0 && ((p.stamp_mask >> (k)) & 1)) p.stamps[blockIdx.x * 16 + (k)] = gtime(); } while (0)

// A wait that has run out once makes every later wait of the block short: the block still runs to its end (its
// output is then meaningless and the host sees the error word) without spending the long bound again and again.
__device__ __forceinline__ void wait_or_give_up(uint64_t* bar, uint32_t parity, volatile int* gave_up, uint32_t* error) {
  if (*gave_up) {
    const uint32_t addr = smem_u32(bar);
    for (int spin = 0; spin < 100000 && !mbar_try(addr, parity); ++spin) {}
    return;
  }
  if (!mbar_wait(bar, parity, error)) *gave_up = 1;
}

// MR: rows of the token operand kept in shared memory (8 or 16).  T8: 8-row groups of weight rows in a sub-tile
// (1, or 2 for SwiGLU: 8 gate rows and their 8 up rows).
//
// Work: sub-tile j holds weight rows [j * 8 * T8, (j + 1) * 8 * T8); block b owns sub-tiles b, b + grid, ...; the
// block's r-th sub-tile goes to warp group r % groups in round r / groups; a group is `ksplit` warps, warp `part` of
// it taking columns [part * kr, (part + 1) * kr) of k.  Every warp is its own pipeline: it copies the rows of its
// next units into its own ring of `depth` stages (a lane per row, one bulk copy per row), waits for a stage, runs
// the MMAs over it and — after its group has added the parts' sums — the first warp of the group stores the result
// straight from its registers.  No barrier of the whole block after the prologue.
template <int MR, int T8, bool NORM, bool SWIGLU, typename NW, typename OT>
__global__ void __launch_bounds__(SK_THREADS, 2) skinny_gemm_kernel(const SkinnyParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int ROWS = 8 * T8;
  const int K = p.K, N = p.N, M = p.M;
  const int LDS = K + SK_X_PAD;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, q = lane & 3;
  const int KS = p.ksplit, depth = p.depth;
  const int group = warp / KS, part = warp % KS;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem) + group * SK_MAX_DEPTH;            // of the warp's group
  uint64_t* xbar = reinterpret_cast<uint64_t*>(smem) + SK_WARPS * SK_MAX_DEPTH;          // the token rows have landed
  volatile int* gave_up = reinterpret_cast<volatile int*>(smem + (SK_WARPS * SK_MAX_DEPTH + 1) * 8);
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem + SK_HEAD_BYTES);            // [MR][LDS]
  const int red_floats = KS > 1 ? 2 * p.groups * (KS - 1) * T8 * 128 : 0;
  float* red = reinterpret_cast<float*>(xs + MR * LDS);                                   // [2][groups][KS - 1][T8 * 128]
  // A stage holds a unit's weight rows as they lie in memory, k after k, row after row: ONE bulk copy brings a unit
  // (a copy costs the SM's copy engine about 40 ns whatever its size; row by row, or part by part, the engine and
  // not the memory set the pace).  Rows are then 2 K bytes apart and the eight rows that a warp reads at once share
  // their banks two by two, which costs a few cycles a load.
  const int row_bytes = K * 2;
  const int stage_bytes = ROWS * row_bytes;
  unsigned char* ring = smem + ((SK_HEAD_BYTES + MR * LDS * 2 + red_floats * 4 + 127) / 128) * 128 +
                        static_cast<size_t>(group) * depth * stage_bytes;

  const int nsub = (N + ROWS - 1) / ROWS;
  const int my_sub = blockIdx.x < nsub ? (nsub - 1 - blockIdx.x) / gridDim.x + 1 : 0;
  const int units = (group < p.groups && my_sub > group) ? (my_sub - 1 - group) / p.groups + 1 : 0;
  const int k_lo = part * p.kr;
  const int cols = max(0, min(p.kr, K - k_lo));            // this part's columns (0: the part lies beyond k)
  STAMP(0);
  if (p.stamps != nullptr && threadIdx.x == 0) p.stamps[blockIdx.x * 16 + 14] = clock64();

  if (part == 0 && lane == 0) {
    for (int d = 0; d < depth; ++d) mbar_init(&full[d], 1);
    if (warp == 0) {
      mbar_init(xbar, 1);
      *gave_up = 0;
    }
    mbar_init_fence();
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // the copy engine sees the barriers as initialised
  }
  __syncwarp();
  const uint64_t policy = evict_first_policy();
  // the copy of the group's unit i into stage i % depth, by the group's first warp: nothing that a kernel writes is
  // read here
  auto issue = [&](int i) {
    if (part != 0) return;
    const int sub = blockIdx.x + (group + i * p.groups) * gridDim.x;
    const int rows = min(ROWS, N - sub * ROWS);
    uint64_t* bar = &full[i % depth];
    unsigned char* dst = ring + (i % depth) * stage_bytes;
    const __nv_bfloat16* src = p.W + static_cast<long long>(sub) * ROWS * p.ldw;
    if (p.ldw == K) {
      if (lane == 0) {
        mbar_expect_tx(bar, static_cast<uint32_t>(rows * row_bytes));
        bulk_copy(dst, src, static_cast<uint32_t>(rows * row_bytes), bar, policy);
      }
    } else {                                               // rows with a gap between them: a copy per row
      if (lane == 0) mbar_expect_tx(bar, static_cast<uint32_t>(rows * row_bytes));
      __syncwarp();
      if (lane < rows) bulk_copy(dst + lane * row_bytes, src + lane * p.ldw, static_cast<uint32_t>(row_bytes), bar, policy);
    }
  };
  if (p.trigger == 2 && threadIdx.x == 0) launch_dependents();
  for (int i = 0; i < min(depth, units); ++i) issue(i);
  // the first group has as many units as any: when its last copy is on its way, so is (about) the block's
  if (p.trigger == 1 && threadIdx.x == 0 && units <= depth) launch_dependents();

  const int chunks16 = K / 8;                              // 16-byte chunks of a token row
  const NW* norm_w = static_cast<const NW*>(p.norm_w);
  constexpr int NWV = 8 * sizeof(NW) / 16;                 // 16-byte loads per 8 norm weights
  uint4 wpre[4][NWV];                                      // norm weights of the lane's first four chunks: no kernel
  if (NORM && my_sub > 0) {                                // writes them either
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = lane + 32 * j;
#pragma unroll
      for (int v = 0; v < NWV; ++v)
        wpre[j][v] = c < chunks16 ? ldg_nc16(reinterpret_cast<const uint4*>(norm_w + c * 8) + v) : make_uint4(0, 0, 0, 0);
    }
  }
  // rows beyond the batch are zero (nothing to wait for)
  for (int row = M + warp; row < MR; row += SK_WARPS) {
    __nv_bfloat16* xrow = xs + row * LDS;
    for (int c = lane; c < chunks16; c += 32) *reinterpret_cast<uint4*>(xrow + c * 8) = make_uint4(0, 0, 0, 0);
  }
  // The residual values that the epilogue of unit i adds; asked for early, they arrive while other work runs.
  // MR == 8: the lane's outputs are weight rows gid, gid + 8 of the unit for tokens 2 q, 2 q + 1 (see the product);
  // MR == 16: tokens gid, gid + 8 at columns 2 q, 2 q + 1.
  float res[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  auto load_residual = [&](int i) {
    if (SWIGLU || p.residual == nullptr || part != 0 || i >= units) return;
    const int n0 = (blockIdx.x + (group + i * p.groups) * gridDim.x) * ROWS;
    if constexpr (MR == 8) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int tok = 2 * q + (e & 1), col = n0 + gid + 8 * (e >> 1);
        if (tok < M && col < N && (e < 2 || T8 == 2)) res[e] = __bfloat162float(p.residual[tok * p.ldo + col]);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int tok = gid + 8 * (e >> 1), col = n0 + 2 * q + (e & 1);
        if (tok < M && col < N) res[e] = __bfloat162float(p.residual[tok * p.ldo + col]);
      }
    }
  };
  wait_for_prior_kernels();
  STAMP(1);
  if (my_sub == 0) return;
  load_residual(0);
  if (p.delta == nullptr) {
    // The token rows: one bulk copy for all of them (with loads through registers a row of 3072 columns took three
    // trips to the L2, one after the other).  Every block of the kernel asks for the same few KB at the same
    // moment, so this trip is the slowest part of a block's life.
    if (warp == 0) {
      if (lane == 0) mbar_expect_tx(xbar, static_cast<uint32_t>(M * K * 2));
      __syncwarp();
      if (p.ldx == K) {
        if (lane == 0) bulk_copy_keep(xs, p.x, static_cast<uint32_t>(M * K * 2), xbar);
      } else if (lane < M) {
        bulk_copy_keep(xs + lane * LDS, p.x + lane * p.ldx, static_cast<uint32_t>(K * 2), xbar);
      }
    }
    wait_or_give_up(xbar, 0, gave_up, p.error);
    STAMP(8);
    if (NORM) {
      // warp w norms rows w, w + 8 in place.  The work is a few hundred dependent instructions of one warp, on every
      // block's path: a lane's four chunks are loaded together, their squares go to four sums of their own, and when
      // a row is one such group (k <= 1024) the values stay in registers between the two passes.
      for (int row = warp; row < M; row += SK_WARPS) {
        __nv_bfloat16* xrow = xs + row * LDS;
        float s4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        uint4 v[4];
        for (int c0 = 0; c0 < chunks16; c0 += 128) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int c = c0 + lane + 32 * j;
            v[j] = c < chunks16 ? *reinterpret_cast<const uint4*>(xrow + c * 8) : make_uint4(0, 0, 0, 0);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const __nv_bfloat162* ve = reinterpret_cast<const __nv_bfloat162*>(&v[j]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = __bfloat1622float2(ve[e]);
              s4[j] = fmaf(f.x, f.x, s4[j]);
              s4[j] = fmaf(f.y, f.y, s4[j]);
            }
          }
        }
        STAMP(10);
        const float ss = warp_sum((s4[0] + s4[1]) + (s4[2] + s4[3]));
        const float scale = 1.0f / sqrtf(ss / static_cast<float>(K) + p.eps);
        if (scale > 0.0f) STAMP(11);
        for (int c0 = 0; c0 < chunks16; c0 += 128) {
          if (chunks16 > 128) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int c = c0 + lane + 32 * j;
              v[j] = c < chunks16 ? *reinterpret_cast<const uint4*>(xrow + c * 8) : make_uint4(0, 0, 0, 0);
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int c = c0 + lane + 32 * j;
            if (c >= chunks16) continue;
            uint4 wq[NWV];
#pragma unroll
            for (int u = 0; u < NWV; ++u)
              wq[u] = c0 == 0 ? wpre[j][u] : ldg_nc16(reinterpret_cast<const uint4*>(norm_w + c * 8) + u);
            const NW* we = reinterpret_cast<const NW*>(wq);
            __nv_bfloat16* ve = reinterpret_cast<__nv_bfloat16*>(&v[j]);
#pragma unroll
            for (int e = 0; e < 8; ++e)
              ve[e] = __float2bfloat16_rn((__bfloat162float(ve[e]) * scale) * to_float<NW>(we[e]));
            *reinterpret_cast<uint4*>(xrow + c * 8) = v[j];
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
      __nv_bfloat16* xrow = xs + row * LDS;
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
        for (int c0 = 0; c0 < chunks16; c0 += 128) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int c = c0 + lane + 32 * j;
            if (c >= chunks16) continue;
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
  }
  STAMP(9);
  __syncthreads();
  STAMP(2);

  OT* out = static_cast<OT*>(p.out);
  const unsigned char* xa = reinterpret_cast<const unsigned char*>(xs) + gid * LDS * 2 + q * 16 + k_lo * 2;
  const int nkb = cols / 32;
  constexpr int CH = MR == 8 ? 8 : 8 / T8;                 // chains of accumulators
  constexpr int NS = MR == 8 ? 1 : T8;                     // accumulator tiles of a unit
  for (int i = 0; i < units; ++i) {
    const int sub = blockIdx.x + (group + i * p.groups) * gridDim.x;
    const int n0 = sub * ROWS;
    wait_or_give_up(&full[i % depth], (i / depth) & 1, gave_up, p.error);
    if (i == 0) STAMP(3);
    if (i == units - 1) STAMP(4);
    // Several chains of accumulators over the part's k blocks, added at the end: a chain of dependent MMAs is what
    // a warp's unit costs, and mma.sync is slow on this hardware.  A thread reads 16 contiguous bytes of a row per
    // 32-wide k block (the k order inside a block is permuted the same way for both operands, which a dot product
    // does not notice).
    //   MR == 8   the unit's 8 or 16 WEIGHT rows are the 16-row operand and the (at most 8) tokens the 8-column
    //             one: no lane of the MMA is wasted on tokens that do not exist; a lane ends up with weight rows
    //             gid, gid + 8 for tokens 2 q, 2 q + 1;
    //   MR == 16  the 16 tokens are the 16-row operand and each 8 weight rows an 8-column one; a lane ends up with
    //             tokens gid, gid + 8 at columns 2 q, 2 q + 1 of each 8-row group.
    const long long cyc0 = clock64();
    float acc[CH][NS][4];
#pragma unroll
    for (int a = 0; a < CH; ++a)
#pragma unroll
      for (int t = 0; t < NS; ++t) acc[a][t][0] = acc[a][t][1] = acc[a][t][2] = acc[a][t][3] = 0.0f;
    const unsigned char* wb = ring + (i % depth) * stage_bytes + gid * row_bytes + k_lo * 2 + q * 16;
    for (int kb0 = 0; kb0 < nkb; kb0 += CH) {
#pragma unroll
      for (int a = 0; a < CH; ++a) {
        const int kb = kb0 + a;
        if (kb < nkb) {
          const uint4 xlo = *reinterpret_cast<const uint4*>(xa + kb * 64);
          if constexpr (MR == 8) {
            const uint4 wlo = *reinterpret_cast<const uint4*>(wb + kb * 64);
            uint4 whi = make_uint4(0, 0, 0, 0);
            if (T8 == 2) whi = *reinterpret_cast<const uint4*>(wb + 8 * row_bytes + kb * 64);
            mma16816(acc[a][0], wlo.x, whi.x, wlo.y, whi.y, xlo.x, xlo.y);
            mma16816(acc[a][0], wlo.z, whi.z, wlo.w, whi.w, xlo.z, xlo.w);
          } else {
            const uint4 xhi = *reinterpret_cast<const uint4*>(xa + 8 * LDS * 2 + kb * 64);
#pragma unroll
            for (int t = 0; t < T8; ++t) {
              const uint4 w = *reinterpret_cast<const uint4*>(wb + t * 8 * row_bytes + kb * 64);
              mma16816(acc[a][t], xlo.x, xhi.x, xlo.y, xhi.y, w.x, w.y);
              mma16816(acc[a][t], xlo.z, xhi.z, xlo.w, xhi.w, w.z, w.w);
            }
          }
        }
      }
    }
    float sum[NS][4];
#pragma unroll
    for (int t = 0; t < NS; ++t)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = 0.0f;
#pragma unroll
        for (int a = 0; a < CH; ++a) v += acc[a][t][e];
        sum[t][e] = v;
      }
    if (i == 0 && sum[0][0] != 12345.0f) STAMP(12);
    if (i == 0 && sum[0][0] != 12345.0f && p.stamps != nullptr && threadIdx.x == 0) p.stamps[blockIdx.x * 16 + 7] = clock64() - cyc0;
    if (KS == 1) {
      // the stage has been read (the sums depend on every load): the group's next unit may land in it
      __syncwarp();
      if (i + depth < units) {
        issue(i + depth);
        if (p.trigger == 1 && threadIdx.x == 0 && i + depth == units - 1) launch_dependents();
      }
    }
    if (KS > 1) {
      // the parts of a sub-tile are added in the order of the parts, by the group's first warp
      float* slot = red + (((i & 1) * p.groups + group) * (KS - 1)) * (T8 * 128);
      if (part > 0) {
#pragma unroll
        for (int t = 0; t < NS; ++t)
          *reinterpret_cast<float4*>(slot + ((part - 1) * T8 + t) * 128 + lane * 4) =
              make_float4(sum[t][0], sum[t][1], sum[t][2], sum[t][3]);
      }
      asm volatile("bar.sync %0, %1;\n" ::"r"(1 + group), "r"(32 * KS) : "memory");
      if (i + depth < units) {                             // every part has read the stage: the next unit may land in it
        issue(i + depth);
        if (p.trigger == 1 && threadIdx.x == 0 && i + depth == units - 1) launch_dependents();
      }
      if (part == 0) {
        for (int pp = 1; pp < KS; ++pp)
#pragma unroll
          for (int t = 0; t < NS; ++t) {
            const float4 v = *reinterpret_cast<const float4*>(slot + ((pp - 1) * T8 + t) * 128 + lane * 4);
            sum[t][0] += v.x;
            sum[t][1] += v.y;
            sum[t][2] += v.z;
            sum[t][3] += v.w;
          }
      }
    }
    if (i == 0 && sum[0][0] != 12345.0f) STAMP(13);
    if (part != 0) continue;
    const float res_now[4] = {res[0], res[1], res[2], res[3]};
    load_residual(i + 1);
    // epilogue, from the registers
    if constexpr (MR == 8) {
      if (SWIGLU) {
        // rows 0..7 of the unit are gate rows, rows 8..15 their up rows: the lane holds both for tokens 2 q, 2 q + 1
        const int col = n0 / 2 + gid;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int tok = 2 * q + e;
          if (tok >= M || col >= N / 2) continue;
          const float g = __bfloat162float(__float2bfloat16_rn(sum[0][e]));
          const float u = __bfloat162float(__float2bfloat16_rn(sum[0][2 + e]));
          out[tok * p.ldo + col] = from_float<OT>((g / (1.0f + expf(-g))) * u);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int tok = 2 * q + (e & 1), col = n0 + gid + 8 * (e >> 1);
          if (tok >= M || col >= N || (e >= 2 && T8 == 1)) continue;
          float o = sum[0][e];
          if (p.residual != nullptr) o = __bfloat162float(__float2bfloat16_rn(o)) + res_now[e];
          out[tok * p.ldo + col] = from_float<OT>(o);
        }
      }
    } else {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int tok = gid + 8 * h;
        if (tok >= M) continue;
        if (SWIGLU) {
          // group 0 of the unit: 8 gate rows, group 1: their 8 up rows -> 8 output columns
          const int col = n0 / 2 + 2 * q;
          float o2[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float g = __bfloat162float(__float2bfloat16_rn(sum[0][2 * h + e]));
            const float u = __bfloat162float(__float2bfloat16_rn(sum[T8 - 1][2 * h + e]));
            o2[e] = (g / (1.0f + expf(-g))) * u;
          }
          OT* dst = out + tok * p.ldo + col;
          if (p.ldo % 2 == 0 && col + 1 < N / 2) {
            if constexpr (sizeof(OT) == 2) *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(o2[0], o2[1]);
            else *reinterpret_cast<float2*>(dst) = make_float2(o2[0], o2[1]);
          } else {
            if (col < N / 2) dst[0] = from_float<OT>(o2[0]);
            if (col + 1 < N / 2) dst[1] = from_float<OT>(o2[1]);
          }
        } else {
#pragma unroll
          for (int t = 0; t < T8; ++t) {
            const int col = n0 + t * 8 + 2 * q;
            float o2[2] = {sum[t][2 * h], sum[t][2 * h + 1]};
            if (p.residual != nullptr && t == 0) {
              o2[0] = __bfloat162float(__float2bfloat16_rn(o2[0])) + res_now[2 * h];
              o2[1] = __bfloat162float(__float2bfloat16_rn(o2[1])) + res_now[2 * h + 1];
            }
            OT* dst = out + tok * p.ldo + col;
            if (p.ldo % 2 == 0 && col + 1 < N) {
              if constexpr (sizeof(OT) == 2) *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(o2[0], o2[1]);
              else *reinterpret_cast<float2*>(dst) = make_float2(o2[0], o2[1]);
            } else {
              if (col < N) dst[0] = from_float<OT>(o2[0]);
              if (col + 1 < N) dst[1] = from_float<OT>(o2[1]);
            }
          }
        }
      }
    }
  }
  if (warp == 0) STAMP(5);
  if (p.stamps != nullptr && threadIdx.x == 0) p.stamps[blockIdx.x * 16 + 15] = clock64();
}

struct SkinnyPlan {
  int grid, ksplit, kr, depth, groups, smem;
};

// How a product of these sizes is cut (see the kernel): one block per SM; the warps that share a sub-tile's k so
// that no warp's chain of k blocks is longer than SK_KR_MAX columns; rings only for the warp groups that have work,
// as deep as the rounds of the busiest block, within about half of an SM's shared memory when the block has few
// rounds (so that the next kernel's block fits beside it) and within most of it when it has many.
template <int MR, int T8>
static bool skinny_plan(int N, int K, int sms, SkinnyPlan* plan) {
  const int rows = 8 * T8;
  const int nsub = (N + rows - 1) / rows;
  plan->grid = nsub < sms ? nsub : sms;
  const int per_block = (nsub + plan->grid - 1) / plan->grid;        // sub-tiles of the busiest block
  const int unit = rows * K * 2;
  // As many warps share a sub-tile's k as leaves every sub-tile of the block a group of its own — all eight warps
  // of a block with one sub-tile, pairs in a block with four — but parts of at least 128 columns, and at most
  // SK_KR_MAX columns a part where k is long; and the groups' stages have to fit into an SM's shared memory.
  int ks = 1;
  while (ks < SK_WARPS && per_block * ks * 2 <= SK_WARPS && K / (ks * 2) >= 128) ks *= 2;
  while (ks < SK_WARPS && (K + ks - 1) / ks > SK_KR_MAX) ks *= 2;
  while (ks < SK_WARPS && MR * K * 2 + (SK_WARPS / ks) * unit > 200 * 1024 && per_block > SK_WARPS / (2 * ks)) ks *= 2;
  plan->ksplit = ks;
  plan->kr = ((K + ks - 1) / ks + 31) / 32 * 32;
  const int wg = SK_WARPS / plan->ksplit;
  plan->groups = per_block < wg ? per_block : wg;
  while (plan->groups > 1 && MR * K * 2 + plan->groups * unit > 200 * 1024) --plan->groups;
  const int rounds = (per_block + plan->groups - 1) / plan->groups;
  const int red = plan->ksplit > 1 ? 2 * plan->groups * (plan->ksplit - 1) * T8 * 512 : 0;
  const int head = ((SK_HEAD_BYTES + MR * (K + SK_X_PAD) * 2 + red + 127) / 128) * 128;
  const int budget = (rounds > 2 ? 200 : 120) * 1024;
  int depth = 1;
  while (depth < SK_MAX_DEPTH && depth < rounds && head + (depth + 1) * plan->groups * unit <= budget) ++depth;
  plan->depth = depth;
  plan->smem = head + depth * plan->groups * unit;
  return plan->smem <= 227 * 1024;
}

int g_knob_trigger = 1, g_knob_target_kb = 108, g_knob_grid = 0;
unsigned long long* g_stamps = nullptr;
int g_stamp_idx = 0;

template <int MR, int T8, bool NORM, bool SWIGLU, typename NW, typename OT = __nv_bfloat16>
static int launch_skinny(SkinnyParams p, cudaStream_t s) {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  SkinnyPlan plan;
  if (!skinny_plan<MR, T8>(p.N, p.K, sms, &plan)) return PIH_ERR_UNSUPPORTED;
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
  if (plan.smem > 48 * 1024 && smem_set < plan.smem) {
    cudaError_t e = cudaFuncSetAttribute(skinny_gemm_kernel<MR, T8, NORM, SWIGLU, NW, OT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, plan.smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    smem_set = plan.smem;
  }
  p.ksplit = plan.ksplit;
  p.kr = plan.kr;
  p.depth = plan.depth;
  p.groups = plan.groups;
  p.trigger = g_knob_trigger;
  p.stamp_mask = g_knob_target_kb;
  p.stamps = g_stamps ? g_stamps + static_cast<size_t>(g_stamp_idx++) * 512 * 16 : nullptr;
  launch_kernel(skinny_gemm_kernel<MR, T8, NORM, SWIGLU, NW, OT>, dim3(plan.grid), dim3(SK_THREADS), plan.smem, s, p);
  if (g_knob_grid == 777) {                                // debug: the same launch once more, with warm caches
    p.stamps = g_stamps ? g_stamps + static_cast<size_t>(g_stamp_idx++) * 512 * 16 : nullptr;
    launch_kernel(skinny_gemm_kernel<MR, T8, NORM, SWIGLU, NW, OT>, dim3(plan.grid), dim3(SK_THREADS), plan.smem, s, p);
  }
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

static bool skinny_takes(const void* x, const void* W, int M, int K, long long ldx, long long ldw) {
  return M <= 16 && K > 0 && K % 32 == 0 && ldx % 8 == 0 && ldw % 8 == 0 &&
         (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(W) & 15) == 0;
}

}  // namespace pih

using namespace pih;

extern "C" int pih_debug_stamps(unsigned long long* buf) {
  g_stamps = buf;
  const int n = g_stamp_idx;
  g_stamp_idx = 0;
  return n;
}
extern "C" int pih_debug_stamp_next() { return g_stamp_idx++; }

extern "C" int pih_debug_knob(int which, int value) {
  int* k = which == 0 ? &g_knob_trigger : which == 1 ? &g_knob_target_kb : &g_knob_grid;
  const int before = *k;
  *k = value;
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
      (reinterpret_cast<uintptr_t>(norm_w) & 15) || (reinterpret_cast<uintptr_t>(out) & 3) ||
      (reinterpret_cast<uintptr_t>(residual) & 3) || residual == out ||
      (delta != nullptr && ((reinterpret_cast<uintptr_t>(delta) & 15) || x_out == nullptr || x_out == x)))
    return PIH_ERR_UNSUPPORTED;
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
  if (!skinny_takes(x, W, M, K, ldx, ldw) || (reinterpret_cast<uintptr_t>(out) & 7)) return PIH_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  SkinnyParams p = {};
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.W = static_cast<const __nv_bfloat16*>(W);
  p.out = out;
  p.M = M, p.N = N, p.K = K;
  p.ldx = ldx, p.ldw = ldw, p.ldo = ldo;
  p.error = error;
  if (M <= 8)
    return N >= 148 * 16 ? launch_skinny<8, 2, false, false, float, float>(p, s)
                         : launch_skinny<8, 1, false, false, float, float>(p, s);
  return launch_skinny<16, 1, false, false, float, float>(p, s);
}
