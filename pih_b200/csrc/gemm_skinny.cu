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
__device__ __forceinline__ uint64_t evict_first_policy() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(p));
  return p;
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 256;\n" ::: "memory"); }

constexpr int SK_WARPS = 8;                      // consumer warps
constexpr int SK_THREADS = (SK_WARPS + 1) * 32;  // and the producer warp
constexpr int SK_KC_MAX = 2048;                  // most columns of a stage: a row of a stage is ONE bulk copy of up to 4 KB
constexpr int SK_MAX_STAGES = 16;
constexpr int SK_X_PAD = 32;                     // elements: the same for the token rows
constexpr int SK_HEAD_BYTES = 512;               // barriers and the give-up flag

struct SkinnyParams {
  const __nv_bfloat16* x;
  const __nv_bfloat16* delta;
  __nv_bfloat16* x_out;
  const void* norm_w;
  const __nv_bfloat16* W;
  void* out;
  float eps;
  int M, N, K;
  long long ldx, ldw, ldo;
  int stages;                                    // of the ring
  int kc, nchunks;                               // columns of a stage (a multiple of 64), stages per tile
  uint32_t* error;
  int trigger;                                   // 0 none, 1 after the last issue, 2 at the top
  unsigned long long* stamps;                    // debug: [8] per block
};
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define STAMP(k) do { if (p.stamps != nullptr && lane == 0 && (warp == 0 || warp == SK_WARPS)) p.stamps[blockIdx.x * 16 + (k)] = gtime(); } while (0)

// MR: rows of the token operand kept in shared memory (8 or 16).  TN: weight rows of a tile (8 or 16).
template <int MR, int TN, bool NORM, bool SWIGLU, typename NW, typename OT>
__global__ void __launch_bounds__(SK_THREADS, 2) skinny_gemm_kernel(const SkinnyParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int T8 = TN / 8;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty = full + SK_MAX_STAGES;
  volatile int* gave_up = reinterpret_cast<volatile int*>(smem + 2 * SK_MAX_STAGES * 8);
  const int K = p.K, N = p.N, M = p.M;
  const int LDS = K + SK_X_PAD;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem + SK_HEAD_BYTES);            // [MR][LDS]
  float* red = reinterpret_cast<float*>(xs + MR * LDS);                                   // [SK_WARPS][T8][16 * 8]
  unsigned char* ring = smem + ((SK_HEAD_BYTES + MR * LDS * 2 + SK_WARPS * T8 * 512 + 127) / 128) * 128;
  const int S = p.stages;
  const int KC = p.kc, nchunks = p.nchunks;
  const int row_bytes = KC * 2 + 64;                       // a stage's rows alternate between the halves of the 128-byte bank window
  const int stage_bytes = TN * row_bytes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ntiles = (N + TN - 1) / TN;
  const int my_tiles = blockIdx.x < ntiles ? (ntiles - 1 - blockIdx.x) / gridDim.x + 1 : 0;
  const int total = my_tiles * nchunks;                    // stages this block streams
  if (warp == 0) STAMP(0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], SK_WARPS);
    }
    *gave_up = 0;
    mbar_init_fence();
  }
  __syncthreads();

  if (warp == SK_WARPS) {
    // ---- producer warp: streams the block's weights through the ring, a lane per weight row and a bulk copy per
    // row of a stage (issued one after the other by one thread, copies of 1 KB took 36 ns each: less than an SM's
    // share of the memory bandwidth).  It reads nothing that a kernel writes, so it never waits for the kernel
    // before this one.
    if (p.trigger == 2 && lane == 0) launch_dependents();
    const uint64_t policy = evict_first_policy();
    int issued = 0;
    for (int i = 0; i < total; ++i) {
      const int s = i % S, round = i / S;
      int ok = 1;
      if (round > 0) {
        if (lane == 0) ok = !*gave_up && mbar_wait(&empty[s], (round - 1) & 1, p.error);
        ok = __shfl_sync(0xffffffffu, ok, 0);
      }
      if (!ok) {
        if (lane == 0) *gave_up = 1;
        break;
      }
      const int tile = blockIdx.x + (i / nchunks) * gridDim.x, c = i % nchunks;
      const int cols = min(KC, K - c * KC);
      const int rows = min(TN, N - tile * TN);
      if (lane == 0) mbar_expect_tx(&full[s], static_cast<uint32_t>(rows * cols * 2));
      __syncwarp();
      if (lane < rows)
        bulk_copy(ring + s * stage_bytes + lane * row_bytes,
                  p.W + (static_cast<long long>(tile) * TN + lane) * p.ldw + c * KC, static_cast<uint32_t>(cols * 2),
                  &full[s], policy);
      issued = i + 1;
    }
    __syncwarp();
    if (lane == 0) {
      if (p.trigger == 1) launch_dependents();             // the block's last weight load is on its way
      STAMP(6);
      if (*gave_up) {
        // the consumers have stopped waiting: the copies still in flight must land before the block may return
        for (int i = max(0, issued - S); i < issued; ++i) mbar_wait(&full[i % S], (i / S) & 1, p.error);
      }
    }
  } else {
    // ---- consumers
    const int gid = lane >> 2, q = lane & 3;
    const int chunks16 = K / 8;                            // 16-byte chunks of a token row
    const NW* norm_w = static_cast<const NW*>(p.norm_w);
    constexpr int NWV = 8 * sizeof(NW) / 16;               // 16-byte loads per 8 norm weights
    uint4 wpre[4][NWV];                                    // norm weights of the lane's first four chunks: no kernel
    if (NORM && total > 0) {                               // writes them either
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = lane + 32 * j;
#pragma unroll
        for (int v = 0; v < NWV; ++v)
          wpre[j][v] = c < chunks16 ? ldg_nc16(reinterpret_cast<const uint4*>(norm_w + c * 8) + v) : make_uint4(0, 0, 0, 0);
      }
    }
    wait_for_prior_kernels();
    STAMP(1);
    if (total > 0) {
      // prologue, once per block: warp w prepares token rows w, w + 8.  A lane takes chunks lane, lane + 32, ...,
      // four at a time with their loads issued together; the residual sum is rounded and kept (one block writes
      // it out), its squares are summed on the way, and the normed row replaces it in shared memory.
      for (int row = warp; row < MR; row += SK_WARPS) {
        __nv_bfloat16* xrow = xs + row * LDS;
        if (row >= M) {
          for (int c = lane; c < chunks16; c += 32) *reinterpret_cast<uint4*>(xrow + c * 8) = make_uint4(0, 0, 0, 0);
          continue;
        }
        float ss = 0.0f;
        for (int c0 = 0; c0 < chunks16; c0 += 128) {
          uint4 v[4], d[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int c = c0 + lane + 32 * j;
            v[j] = d[j] = make_uint4(0, 0, 0, 0);
            if (c < chunks16) {
              v[j] = *reinterpret_cast<const uint4*>(p.x + row * p.ldx + c * 8);
              if (p.delta != nullptr) d[j] = *reinterpret_cast<const uint4*>(p.delta + row * p.ldx + c * 8);
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int c = c0 + lane + 32 * j;
            if (c >= chunks16) continue;
            __nv_bfloat16* ve = reinterpret_cast<__nv_bfloat16*>(&v[j]);
            if (p.delta != nullptr) {
              const __nv_bfloat16* de = reinterpret_cast<const __nv_bfloat16*>(&d[j]);
#pragma unroll
              for (int e = 0; e < 8; ++e) ve[e] = __float2bfloat16_rn(__bfloat162float(ve[e]) + __bfloat162float(de[e]));
              // the sum goes to a buffer of its own: other blocks are still reading x
              if (blockIdx.x == 0) *reinterpret_cast<uint4*>(p.x_out + row * p.ldx + c * 8) = v[j];
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
        STAMP(8);
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
      STAMP(9);
      consumer_sync();
      STAMP(2);

      OT* out = static_cast<OT*>(p.out);
      const unsigned char* xa = reinterpret_cast<const unsigned char*>(xs) + gid * LDS * 2 + q * 16;
      float acc[T8][4];
      for (int i = 0; i < total; ++i) {
        const int s = i % S, c = i % nchunks;
        if (c == 0) {
#pragma unroll
          for (int t = 0; t < T8; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.0f;
        }
        if (*gave_up || !mbar_wait(&full[s], (i / S) & 1, p.error)) *gave_up = 1;
        if (i == 0) STAMP(3);
        if (i == total - 1) STAMP(4);
        const unsigned char* wb = ring + s * stage_bytes + gid * row_bytes + q * 16;
        const int blocks = min(KC, K - c * KC) / 32;
        for (int kb = warp; kb < blocks; kb += SK_WARPS) {
          const unsigned char* xk = xa + (c * KC + kb * 32) * 2;
          const uint4 xlo = *reinterpret_cast<const uint4*>(xk);
          uint4 xhi = make_uint4(0, 0, 0, 0);
          if (MR == 16) xhi = *reinterpret_cast<const uint4*>(xk + 8 * LDS * 2);
#pragma unroll
          for (int t = 0; t < T8; ++t) {
            const uint4 w = *reinterpret_cast<const uint4*>(wb + t * 8 * row_bytes + kb * 64);
            mma16816(acc[t], xlo.x, xhi.x, xlo.y, xhi.y, w.x, w.y);
            mma16816(acc[t], xlo.z, xhi.z, xlo.w, xhi.w, w.z, w.w);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);             // this warp has read what it needs of the stage
        if (c != nchunks - 1) continue;
        // the tile is complete: the warps' partial sums, added in warp order
        const int tile = blockIdx.x + (i / nchunks) * gridDim.x;
        const int n0 = tile * TN;
#pragma unroll
        for (int t = 0; t < T8; ++t) {
          float* r = red + (warp * T8 + t) * 128;
          r[gid * 8 + q * 2] = acc[t][0];
          r[gid * 8 + q * 2 + 1] = acc[t][1];
          r[(gid + 8) * 8 + q * 2] = acc[t][2];
          r[(gid + 8) * 8 + q * 2 + 1] = acc[t][3];
        }
        consumer_sync();
        if (SWIGLU) {
          // rows 0..7 of the tile: 8 gate rows, rows 8..15: their 8 up rows -> 8 output columns
          const int tok = threadIdx.x >> 3, col = threadIdx.x & 7;
          if (threadIdx.x < 128 && tok < M && n0 / 2 + col < N / 2) {
            float g = 0.0f, u = 0.0f;
#pragma unroll
            for (int w = 0; w < SK_WARPS; ++w) {
              g += red[(w * T8 + 0) * 128 + tok * 8 + col];
              u += red[(w * T8 + (T8 - 1)) * 128 + tok * 8 + col];
            }
            g = __bfloat162float(__float2bfloat16_rn(g));
            u = __bfloat162float(__float2bfloat16_rn(u));
            out[tok * p.ldo + n0 / 2 + col] = from_float<OT>((g / (1.0f + expf(-g))) * u);
          }
        } else {
          for (int e = threadIdx.x; e < T8 * 128; e += SK_WARPS * 32) {
            const int t = e >> 7, tok = (e & 127) >> 3, col = e & 7;
            if (tok < M && n0 + t * 8 + col < N) {
              float sum = 0.0f;
#pragma unroll
              for (int w = 0; w < SK_WARPS; ++w) sum += red[(w * T8 + t) * 128 + tok * 8 + col];
              out[tok * p.ldo + n0 + t * 8 + col] = from_float<OT>(sum);
            }
          }
        }
        consumer_sync();                                   // red is reused by the next tile
      }
    }
  }
  __syncthreads();                                         // nobody returns while a copy may still land in the ring
  if (warp == 0) STAMP(5);
}

// Columns of a stage: the tile's whole k when that is at most SK_KC_MAX, else k cut into equal parts; a multiple of 64
// so that a stage's rows alternate between the halves of the bank window.
static void skinny_chunks(int K, int* kc, int* nchunks) {
  *nchunks = (K + SK_KC_MAX - 1) / SK_KC_MAX;
  *kc = ((K + *nchunks - 1) / *nchunks + 63) / 64 * 64;
  *nchunks = (K + *kc - 1) / *kc;
}

// Shared memory of a launch: the token rows, the partial sums and a ring of `stages` stages.
template <int MR, int TN>
static int skinny_smem(int K, int stages) {
  int kc, nchunks;
  skinny_chunks(K, &kc, &nchunks);
  const int head = ((SK_HEAD_BYTES + MR * (K + SK_X_PAD) * 2 + SK_WARPS * (TN / 8) * 512 + 127) / 128) * 128;
  return head + stages * TN * (kc * 2 + 64);
}

int g_knob_trigger = 1, g_knob_target_kb = 108, g_knob_grid = 0;
unsigned long long* g_stamps = nullptr;
int g_stamp_idx = 0;

template <int MR, int TN, bool NORM, bool SWIGLU, typename NW, typename OT = __nv_bfloat16>
static int launch_skinny(SkinnyParams p, cudaStream_t s) {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  const int ntiles = (p.N + TN - 1) / TN;
  const int cap = g_knob_grid > 0 ? g_knob_grid : sms;
  const int grid = ntiles < cap ? ntiles : cap;
  skinny_chunks(p.K, &p.kc, &p.nchunks);
  const int most = ((ntiles + grid - 1) / grid) * p.nchunks;        // stages of the busiest block
  // As many stages as bring the block to about 108 KB, so that the next kernel's block fits on the SM beside it;
  // a block with many tiles to walk over (the output head) runs for long and takes what it needs to keep an SM's
  // share of the bandwidth in flight instead.
  const int kTarget = (most > 6 ? 200 : g_knob_target_kb) * 1024;
  p.trigger = g_knob_trigger;
  p.stamps = g_stamps ? g_stamps + static_cast<size_t>(g_stamp_idx++) * 512 * 16 : nullptr;
  int stages = 2;
  while (stages < SK_MAX_STAGES && stages < most && skinny_smem<MR, TN>(p.K, stages + 1) <= kTarget) ++stages;
  const int smem = skinny_smem<MR, TN>(p.K, stages);
  if (smem > 227 * 1024) return PIH_ERR_UNSUPPORTED;
  static int smem_set = 0;                                 // per instance
  if (smem > 48 * 1024 && smem_set < smem) {
    cudaError_t e = cudaFuncSetAttribute(skinny_gemm_kernel<MR, TN, NORM, SWIGLU, NW, OT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    smem_set = smem;
  }
  p.stages = stages;
  launch_kernel(skinny_gemm_kernel<MR, TN, NORM, SWIGLU, NW, OT>, dim3(grid), dim3(SK_THREADS), smem, s, p);
  PIH_LAUNCH_CHECK();
  return 0;
}

template <int MR, bool NORM, typename NW>
static int dispatch_skinny(bool tall, bool swiglu, const SkinnyParams& p, cudaStream_t s) {
  if (swiglu) return launch_skinny<MR, 16, NORM, true, NW>(p, s);
  if (tall) return launch_skinny<MR, 16, NORM, false, NW>(p, s);
  return launch_skinny<MR, 8, NORM, false, NW>(p, s);
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
//   error      the device's error word (a bounded wait that ran out is reported there)
// Returns PIH_ERR_UNSUPPORTED for shapes it does not take (the caller uses the separate kernels).
extern "C" int pih_gemm_skinny(const void* x, const void* delta, void* x_out, int norm_dtype, const void* norm_w,
                               float eps, const void* W, void* out, int M, int N, int K, long long ldx,
                               long long ldw, long long ldo, int swiglu, uint32_t* error, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (!skinny_takes(x, W, M, K, ldx, ldw) || (swiglu && N % 16) || (reinterpret_cast<uintptr_t>(norm_w) & 15) ||
      (delta != nullptr && ((reinterpret_cast<uintptr_t>(delta) & 15) || x_out == nullptr || x_out == x)))
    return PIH_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  SkinnyParams p = {static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(delta),
                    static_cast<__nv_bfloat16*>(x_out), norm_w, static_cast<const __nv_bfloat16*>(W), out, eps,
                    M, N, K, ldx, ldw, ldo, 0, 0, 0, error};
  // 16 weight rows per tile when that still gives every SM a tile, else 8
  const bool tall = N >= 148 * 16;
  const bool sw = swiglu != 0;
#define PIH_SKINNY(MR, NORM, NW) dispatch_skinny<MR, NORM, NW>(tall, sw, p, s)
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
  SkinnyParams p = {static_cast<const __nv_bfloat16*>(x), nullptr, nullptr, nullptr,
                    static_cast<const __nv_bfloat16*>(W), out, 0.0f, M, N, K, ldx, ldw, ldo, 0, 0, 0, error};
  const bool tall = N >= 148 * 16;
#define PIH_SKINNY_F32(MR, TN) launch_skinny<MR, TN, false, false, float, float>(p, s)
  if (tall) return M <= 8 ? PIH_SKINNY_F32(8, 16) : PIH_SKINNY_F32(16, 16);
  return M <= 8 ? PIH_SKINNY_F32(8, 8) : PIH_SKINNY_F32(16, 8);
#undef PIH_SKINNY_F32
}
