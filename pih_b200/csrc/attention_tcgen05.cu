// Causal grouped-query attention of prompt portions on the 5th-generation tensor cores: S = Q K^T and
// O += P V are tcgen05.mma with S and O in tensor memory; K and V pages come by TMA.
//
// Formula as the reference's kernel (kernels/cuda/qwen_bf16_primitives.cu:660-733): score = (q . k) * scale,
// causal mask by position, online softmax in 32-bit, one rounding of acc / sum.  Execution:
//
//   tile       128 packed rows (token i / G, head g G + i % G) of one (request, kv head) x 128 keys
//   warps 0-7  softmax: a row (= tensor-memory lane) is shared by two threads, one per half of the 128 key
//              columns: each reads its 64 scores once (tcgen05.ld), masks, takes the maximum, and writes P (bf16,
//              packed in pairs) back into tensor memory (tcgen05.st), where the P V product reads it as its A
//              operand: P never passes through shared memory, whose bandwidth the S product alone fills
//              (Q and K tiles: 64 KB per 128 x 128 x 128 product at 128 bytes a cycle).  It keeps its part of the
//              row sum; O in tensor memory is rescaled only when the running maximum grew by more than 2^8
//              (otherwise the old reference maximum stays, which is exact because the final division uses the
//              sum formed with the same reference);
//   warps 8, 10  producers: lane p looks up page p of the key tile and issues its TMA boxes; warp 8 feeds the
//              K ring (three stages), warp 10 the V ring (two);
//   warps 9, 11  a thread each issues the MMAs: warp 9 S_j = Q K_j^T (8 x K=16) into one of two S buffers, warp 11
//              O += P_j V_j from one of two P buffers; S_j overlaps the softmax of tile j-1, and the softmax of
//              tile j never waits for the P V product of tile j-1.
//   A CTA takes a late row tile (many keys) and then its early mirror image (few keys), so CTAs are balanced.
//
// Tensor memory: S0 [0,128) S1 [128,256) O [256, 256 + D) P0 [384,448) P1 [448,512).  Every mbarrier wait is bounded.
// No cluster, no multicast.
#include <string.h>

#include "ptx.cuh"

namespace pih {

constexpr int TQ = 128;                 // packed rows per tile
constexpr int TK = 128;                 // keys per tile
constexpr int K_STAGES = 3;             // K tiles run ahead of the S products,
constexpr int V_STAGES = 2;             // V tiles follow the P V products, each ring fed by a warp of its own
constexpr int P_BUFS = 2;               // P tiles (bf16) in tensor memory
constexpr float kLog2e5 = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;   // log2 units

struct PrefillParams {
  const __nv_bfloat16* q;
  int q_stride;
  __nv_bfloat16* out;
  const int* block_table;
  int table_width;
  const int* cu_q;
  const int* q_start;
  int heads, kv_heads, page_size, page_shift, num_pages;
  int num_requests;
  int pair_above;                      // row tiles x kv heads beyond which a block takes two row tiles
  float scale;
  int window;
  uint32_t* error;
};

// K-major operand tile [rows x 64 bf16] with the 128-byte swizzle: see gemm_tcgen05.cu
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t smem_addr) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  desc |= static_cast<uint64_t>(1) << 16;
  desc |= static_cast<uint64_t>(1024 >> 4) << 32;
  desc |= static_cast<uint64_t>(1) << 46;
  desc |= static_cast<uint64_t>(2) << 61;
  return desc;
}
// MN-major operand (V as B of P V: N = head dim contiguous, K = keys along rows of 128 bytes): panels of 64
// columns are `panel_bytes` apart (leading byte offset), groups of 8 keys 1024 bytes apart (stride byte offset).
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t smem_addr, uint32_t panel_bytes) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  desc |= static_cast<uint64_t>((panel_bytes >> 4) & 0x3FFF) << 16;
  desc |= static_cast<uint64_t>(1024 >> 4) << 32;
  desc |= static_cast<uint64_t>(1) << 46;
  desc |= static_cast<uint64_t>(2) << 61;
  return desc;
}
__host__ __device__ constexpr uint32_t idesc_bf16(int m, int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}
// the same with the A operand (M x 16, 16-bit elements packed in pairs: lane = row, 8 columns) in tensor memory
__device__ __forceinline__ void umma_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                            uint32_t acc) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, uint32_t (&v)[64]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
      "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
      "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];\n"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31]), "=r"(v[32]),
        "=r"(v[33]), "=r"(v[34]), "=r"(v[35]), "=r"(v[36]), "=r"(v[37]), "=r"(v[38]), "=r"(v[39]), "=r"(v[40]),
        "=r"(v[41]), "=r"(v[42]), "=r"(v[43]), "=r"(v[44]), "=r"(v[45]), "=r"(v[46]), "=r"(v[47]), "=r"(v[48]),
        "=r"(v[49]), "=r"(v[50]), "=r"(v[51]), "=r"(v[52]), "=r"(v[53]), "=r"(v[54]), "=r"(v[55]), "=r"(v[56]),
        "=r"(v[57]), "=r"(v[58]), "=r"(v[59]), "=r"(v[60]), "=r"(v[61]), "=r"(v[62]), "=r"(v[63])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
      "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]),
      "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]),
      "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
      "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// 2^x by the special-function unit (ex2.approx: 2 ulp; -inf gives 0)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void cp16(void* smem, const void* gmem, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem), "r"(bytes));
}

// Packed row i of a (request, kv head) is token i / G, head g G + i % G.  A thread that walks rows i, i + step, ...
// keeps the pair up to date with additions: the two divisions are done once (a walk with a division per row
// made one warp's fetch of a Q tile take about ten thousand cycles).
struct PackedRowWalk {
  int i, tok, hd, step, tok_step, hd_step, G;
  __device__ __forceinline__ PackedRowWalk(int first, int step_, int G_)
      : i(first), tok(first / G_), hd(first % G_), step(step_), tok_step(step_ / G_), hd_step(step_ % G_), G(G_) {}
  __device__ __forceinline__ void next() {
    i += step;
    tok += tok_step;
    hd += hd_step;
    if (hd >= G) {
      hd -= G;
      ++tok;
    }
  }
};

// A query tile (TQ packed rows) into shared memory as D / 64 panels of 128 rows x 128 bytes with the 128-byte
// swizzle, by threads t of nthreads (a multiple of D / 8: a thread keeps its 16-byte column); rows past `packed`
// are zero.
template <int D>
__device__ __forceinline__ void load_q_tile(unsigned char* q_smem, const PrefillParams& p, int row0, int g, int G,
                                            int packed, int tile_row0, int t, int nthreads) {
  constexpr int PANEL_BYTES = TQ * 128;
  constexpr int CPR = D / 8;                                     // 16-byte chunks of a row
  const int ch = t % CPR, row_step = nthreads / CPR;
  PackedRowWalk w(tile_row0 + t / CPR, row_step, G);
  unsigned char* col = q_smem + (ch >> 3) * PANEL_BYTES;
  for (int qrow = t / CPR; qrow < TQ; qrow += row_step, w.next()) {
    const bool valid = w.i < packed;
    const __nv_bfloat16* src = p.q;
    if (valid)
      src = p.q + static_cast<size_t>(row0 + w.tok) * p.q_stride + static_cast<size_t>(g * G + w.hd) * D + ch * 8;
    cp16(col + qrow * 128 + (((ch & 7) ^ (qrow & 7)) << 4), src, valid ? 16 : 0);
  }
}

template <int D, int SPLIT>
struct PrefillSmem {
  static constexpr int PANELS = D / 64;
  static constexpr int PANEL_BYTES = TQ * 128;                  // a panel of Q or P: 128 rows x 128 bytes
  static constexpr int KV_PANEL_BYTES = TK * 128;               // a panel of K or V: TK keys x 128 bytes
  alignas(1024) unsigned char q[PANELS * PANEL_BYTES];
  alignas(1024) unsigned char k[K_STAGES][PANELS * KV_PANEL_BYTES];
  alignas(1024) unsigned char v[V_STAGES][PANELS * KV_PANEL_BYTES];
  alignas(8) uint64_t q_full, o_ready, p_full[P_BUFS], p_empty[P_BUFS];
  alignas(8) uint64_t k_full[K_STAGES], k_empty[K_STAGES], v_full[V_STAGES], v_empty[V_STAGES];
  alignas(8) uint64_t s_full[2], s_empty[2], r_full[2];
  float xmax[2][2][SPLIT][128];                                 // [set][parity of the set's tile][column part][row] maxima
  float mref[2][128];                                           // [tile parity][row] the reference maximum after that tile
  float xsum[2 * SPLIT][128];                                   // row sums of the sets' column parts
  uint32_t tmem_base;
};

// Two SETS of softmax warps take the key tiles in turn (set = tile & 1); in a set, SPLIT threads share a row
// (= tensor-memory lane), each with 128 / SPLIT of the key columns and D / SPLIT of the output columns.  Warps
// 0 .. 8 SPLIT - 1 are softmax warps (set 0 first), then the producer and MMA warps.
template <int THREADS> __device__ __forceinline__ void softmax_sync() {
  asm volatile("bar.sync 1, %0;\n" ::"n"(THREADS) : "memory");
}
// the SPLIT warps of a set (w, w + 4, ...) that share tensor-memory lanes 32 quarter .. 32 quarter + 31
template <int THREADS> __device__ __forceinline__ void row_group_sync(int set, int quarter) {
  asm volatile("bar.sync %0, %1;\n" ::"r"(2 + 4 * set + quarter), "n"(THREADS) : "memory");
}
// set 0 alone (the epilogue)
template <int THREADS> __device__ __forceinline__ void first_set_sync() {
  asm volatile("bar.sync 10, %0;\n" ::"n"(THREADS) : "memory");
}

// One CTA works through up to two row tiles of its (request, kv head): a long one (late rows, many keys)
// and its short mirror image, so that every CTA has about the same number of key tiles.
template <int D, int SPLIT>
__global__ void __launch_bounds__(256 * SPLIT + 128)
attn_prefill_tcgen05_kernel(const PrefillParams p, const __grid_constant__ CUtensorMap kv_map) {
  using Smem = PrefillSmem<D, SPLIT>;
  constexpr int kSetThreads = 128 * SPLIT;                        // softmax threads of a set
  constexpr int kSetWarps = 4 * SPLIT;
  constexpr int kSoftmaxThreads = 2 * kSetThreads;
  constexpr int kSoftmaxWarps = 2 * kSetWarps;
  constexpr int kProducerWarp = kSoftmaxWarps, kMmaWarp = kSoftmaxWarps + 1, kProducerWarpV = kSoftmaxWarps + 2;
  constexpr int kMmaWarpPV = kSoftmaxWarps + 3;
  constexpr int CW = TK / SPLIT;                                  // key columns of a softmax thread
  constexpr int OW = D / SPLIT;                                   // output columns of a softmax thread
  static_assert(CW == 64 || CW == 32, "a thread reads its scores with one tcgen05.ld of 32 or 64 columns");
  static_assert(OW % 32 == 0, "a thread rescales and stores its output columns 32 at a time");
  constexpr int PANELS = Smem::PANELS;
  constexpr int PANEL_BYTES = Smem::PANEL_BYTES;
  constexpr int KV_PANEL_BYTES = Smem::KV_PANEL_BYTES;
  extern __shared__ unsigned char smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  // Which rows are this block's: the row tiles of all requests that bring more than 16 packed rows are numbered
  // through, from the step's row ranges on the device (a step's make-up is data, not launch geometry: the grid is
  // an upper bound, and a captured graph serves every make-up).  With many tiles a block takes a late tile and its
  // early mirror image; with few — a portion of a few hundred tokens beside decoding requests — a tile each, so
  // that twice as many SMs work.
  const int g = blockIdx.y;
  const int G = p.heads / p.kv_heads;
  int total_tiles = 0;
  for (int q = 0; q < p.num_requests; ++q) {
    const int pk = (p.cu_q[q + 1] - p.cu_q[q]) * G;
    if (pk > 16) total_tiles += (pk + TQ - 1) / TQ;
  }
  const bool paired = total_tiles * p.kv_heads > p.pair_above;
  int r = -1, bx = static_cast<int>(blockIdx.x);
  for (int q = 0; q < p.num_requests; ++q) {
    const int pk = (p.cu_q[q + 1] - p.cu_q[q]) * G;
    if (pk <= 16) continue;                                     // decode-like: the split kernel's
    const int t = (pk + TQ - 1) / TQ;
    const int mine = paired ? (t + 1) / 2 : t;
    if (bx < mine) {
      r = q;
      break;
    }
    bx -= mine;
  }
  if (r < 0) return;
  const int row0 = p.cu_q[r];
  const int n_tok = p.cu_q[r + 1] - row0;
  const int packed = n_tok * G;
  const int tiles_q = (packed + TQ - 1) / TQ;
  const int items = (paired && 2 * bx < tiles_q - 1) ? 2 : 1;    // the middle tile of an odd count stands alone
  const int start = p.q_start[r];
  const int* table = p.block_table + static_cast<size_t>(r) * p.table_width;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  // Up to here the block has read only what the step's set-up wrote (row ranges, starts: kernels before the one
  // before this, which has waited for them itself) and taken its tensor memory: that ran beside the end of the
  // q/k kernel.  Its q rows and the cache are read from here on.
  wait_for_prior_kernels();
  launch_dependents();                                   // (the next kernel's blocks may become resident and wait)

  for (int item = 0; item < items; ++item) {
    const int qt = item == 0 ? tiles_q - 1 - bx : bx;
    const int tile_row0 = qt * TQ;
    const int tok_lo = tile_row0 / G;
    const int tok_hi = min(packed - 1, tile_row0 + TQ - 1) / G;
    const int kmin = p.window > 0 ? max(0, start + tok_lo - p.window + 1) : 0;
    const int kmax = start + tok_hi;
    const int t_first = kmin / TK, t_last = kmax / TK;
    const int ntiles = t_last - t_first + 1;

    // (re)initialise the barriers: everything of the previous item has completed (its epilogue waited for the
    // last MMA, and every load had been consumed by an MMA)
    if (threadIdx.x == 0) {
      if (item > 0) {
        auto inval = [](uint64_t* bar) {
          asm volatile("mbarrier.inval.shared::cta.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
        };
        inval(&sm.q_full);
        inval(&sm.o_ready);
        for (int s = 0; s < K_STAGES; ++s) {
          inval(&sm.k_full[s]);
          inval(&sm.k_empty[s]);
        }
        for (int s = 0; s < V_STAGES; ++s) {
          inval(&sm.v_full[s]);
          inval(&sm.v_empty[s]);
        }
        for (int b = 0; b < 2; ++b) {
          inval(&sm.s_full[b]);
          inval(&sm.s_empty[b]);
          inval(&sm.r_full[b]);
        }
        for (int b = 0; b < P_BUFS; ++b) {
          inval(&sm.p_full[b]);
          inval(&sm.p_empty[b]);
        }
      }
      // the softmax warps arrive once per warp (lane 0, after the warp has synchronised): 256 arrivals of
      // single threads on one barrier word cost more than the tile's arithmetic
      mbar_init(&sm.q_full, kSoftmaxWarps);
      mbar_init(&sm.o_ready, 1);
      for (int b = 0; b < P_BUFS; ++b) {
        mbar_init(&sm.p_full[b], kSetWarps);                     // buffer b is set b's
        mbar_init(&sm.p_empty[b], 1);
      }
      for (int s = 0; s < K_STAGES; ++s) {
        mbar_init(&sm.k_full[s], 1);
        mbar_init(&sm.k_empty[s], 1);
      }
      for (int s = 0; s < V_STAGES; ++s) {
        mbar_init(&sm.v_full[s], 1);
        mbar_init(&sm.v_empty[s], 1);
      }
      for (int b = 0; b < 2; ++b) {
        mbar_init(&sm.s_full[b], 1);
        mbar_init(&sm.s_empty[b], kSetWarps);
        mbar_init(&sm.r_full[b], 4);                             // the set's warps of column part 0 publish the reference
      }
      mbar_init_fence();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;
    const uint32_t tmem_o = tmem + 256;

    if (warp == kProducerWarp || warp == kProducerWarpV) {
      // ---------------- producers: one warp feeds the K ring, one the V ring ----------------
      // lane p looks up page p of the key tile and issues its TMA boxes; the rings are independent, so a K
      // tile never waits for the P V product that frees a V buffer (with one warp for both, the S product
      // waited 600 cycles a tile for its K)
      const bool is_v = warp == kProducerWarpV;
      const int stages = is_v ? V_STAGES : K_STAGES;
      uint64_t* full = is_v ? sm.v_full : sm.k_full;
      uint64_t* empty = is_v ? sm.v_empty : sm.k_empty;
      unsigned char* ring = is_v ? sm.v[0] : sm.k[0];
      const int pages_per_tile = TK >> p.page_shift;
      const int fallback = kmin >> p.page_shift;
      if (lane == 0 && item == 0) tma_prefetch_map(&kv_map);
      bool alive = true;
      for (int j = 0; j < ntiles && alive; ++j) {
        const int s = j % stages;
        const int use = j / stages;
        int page = 0;
        if (lane < pages_per_tile) {
          const int j_page = (t_first + j) * TK + lane * p.page_size;
          const bool seen = j_page <= kmax && j_page + p.page_size - 1 >= kmin;
          page = table[seen ? (j_page >> p.page_shift) : fallback];
          if (page < 0 || page >= p.num_pages) {
            publish_error(p.error, kRowWithoutPage);
            page = 0;
          }
        }
        if (use > 0) alive = mbar_wait(&empty[s], (use - 1) & 1, p.error);
        alive = __all_sync(0xffffffffu, alive);
        if (!alive) break;
        if (lane == 0) mbar_expect_tx(&full[s], PANELS * KV_PANEL_BYTES);
        __syncwarp();
        if (lane < pages_per_tile) {
          const int z = (page * 2 + (is_v ? 1 : 0)) * p.kv_heads + g;
          unsigned char* dst = ring + s * (PANELS * KV_PANEL_BYTES) + lane * p.page_size * 128;
#pragma unroll
          for (int pn = 0; pn < PANELS; ++pn)
            tma_load_3d(dst + pn * KV_PANEL_BYTES, &kv_map, pn * 64, 0, z, &full[s]);
        }
      }
      if (item == 0 && items == 2) {
        // The mirror tile's Q rows, fetched by the two producer warps while this tile's last steps and its
        // epilogue run (a block of a 2048-token prompt spent 3.3 of its 59 thousand cycles waiting for them).
        // Q is free once the last S product has read it: that product's completion is the last arrival on its
        // K stage's barrier.
        const int jl = ntiles - 1;
        if (alive) alive = mbar_wait(&sm.k_empty[jl % K_STAGES], (jl / K_STAGES) & 1, p.error);
        __syncwarp();
        load_q_tile<D>(sm.q, p, row0, g, G, packed, bx * TQ, (is_v ? 32 : 0) + lane, 64);
        asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
        proxy_fence();                                           // before the barrier that ends the item
      }
    } else if (warp == kMmaWarp) {
      // ---------------- MMA issuer of S_j = Q K_j^T ----------------
      // The S products and the P V products are issued by a thread each.  One thread for both was the block's
      // bottleneck: a tcgen05.mma costs its issuer about 80 cycles, a satisfied barrier wait with its fence
      // about 270, so sixteen MMAs and four waits a tile came to 2750 cycles against 1900 of softmax.
      if (lane == 0) {
        constexpr uint32_t idesc_s = idesc_bf16(TQ, TK, false);
        // Operand descriptors are made once; a descriptor's low bits hold the address in units of 16 bytes, so
        // a step to another k slice, panel or stage is one 64-bit addition.
        uint64_t q_desc[D / 16];
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          q_desc[kk] = desc_kmajor(smem_u32(sm.q) + (kk / 4) * PANEL_BYTES + (kk % 4) * 32);
        const uint64_t k_desc0 = desc_kmajor(smem_u32(sm.k[0]));
        constexpr uint64_t kStageUnits = (PANELS * KV_PANEL_BYTES) >> 4;
        // item 1: its Q tile was in place, and fenced for the tensor core's reads, before the barrier that
        // ended item 0
        bool alive = item > 0 || mbar_wait(&sm.q_full, 0, p.error);
        tc_fence_after();
        for (int j = 0; j < ntiles && alive; ++j) {
          const int b = j & 1, use = j >> 1, s = j % K_STAGES;
          if (use > 0 && !mbar_wait(&sm.s_empty[b], (use - 1) & 1, p.error)) break;
          if (!mbar_wait(&sm.k_full[s], (j / K_STAGES) & 1, p.error)) break;
          tc_fence_after();
          const uint64_t k_desc = k_desc0 + static_cast<uint64_t>(s) * kStageUnits;
          const uint32_t tmem_s = tmem + b * TK;
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)
            umma(tmem_s, q_desc[kk], k_desc + (((kk / 4) * KV_PANEL_BYTES + (kk % 4) * 32) >> 4), idesc_s,
                 kk > 0 ? 1u : 0u);
          umma_commit(&sm.k_empty[s]);
          umma_commit(&sm.s_full[b]);
        }
      }
    } else if (warp == kMmaWarpPV) {
      // ---------------- MMA issuer of O += P_i V_i ----------------
      if (lane == 0) {
        constexpr uint32_t idesc_o = idesc_bf16(TQ, D, true);
        const uint64_t v_desc0 = desc_mnmajor(smem_u32(sm.v[0]), KV_PANEL_BYTES);
        constexpr uint64_t kStageUnits = (PANELS * KV_PANEL_BYTES) >> 4;
        for (int i = 0; i < ntiles; ++i) {
          const int s = i % V_STAGES;
          if (!mbar_wait(&sm.p_full[i % P_BUFS], (i / P_BUFS) & 1, p.error)) break;
          if (!mbar_wait(&sm.v_full[s], (i / V_STAGES) & 1, p.error)) break;
          tc_fence_after();
          const uint64_t v_desc = v_desc0 + static_cast<uint64_t>(s) * kStageUnits;
          const uint32_t tmem_p = tmem + 384 + (i % P_BUFS) * (TK / 2);
#pragma unroll
          for (int kk = 0; kk < TK / 16; ++kk)
            umma_a_tmem(tmem_o, tmem_p + kk * 8, v_desc + ((kk * 16 * 128) >> 4), idesc_o, (i > 0 || kk > 0) ? 1u : 0u);
          umma_commit(&sm.v_empty[s]);
          umma_commit(&sm.p_empty[i % P_BUFS]);
          if (i == ntiles - 1) umma_commit(&sm.o_ready);
        }
      }
    } else {
      // ---------------- softmax / epilogue: two sets of SPLIT threads per row ----------------
      // Set s takes the key tiles j = s, s + 2, ... with S buffer s and P buffer s.  A tile's softmax is a chain of
      // phases (wait for S, read it, maximum, exchange in the row, exponentials, store of P), and only the
      // exponentials use the special-function unit that bounds the tile: with one set all warps are in the same
      // phase and the unit idles half of the time; with two, one set's other phases run under the other set's
      // exponentials.  What the sets share is the row's running reference maximum (a chain through shared memory,
      // published early in a tile) and O, which a set rescales — rarely — between the P V products of the tile
      // before and of its own; each thread keeps its own part of the row sum until the end.
      const int t = threadIdx.x;                                 // 0 .. kSoftmaxThreads - 1
      const int set = warp / kSetWarps;
      const int part = (warp >> 2) % SPLIT;                      // which CW of the 128 key columns (and OW of D)
      const int row = (warp & 3) * 32 + lane;                    // tensor-memory lane
      const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
      if (item == 0) {
        // (the mirror tile's rows were fetched by the K producer while the first tile's last steps ran)
        load_q_tile<D>(sm.q, p, row0, g, G, packed, tile_row0, t, kSoftmaxThreads);
        asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
        proxy_fence();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.q_full);
      }

      const int i_row = tile_row0 + row;
      const bool row_valid = i_row < packed;
      // A row past the request's last (the tile is not full) sees every key, like the tile's full rows far from the
      // diagonal: nothing of it is stored, and it must not put its warp on the masked path in every key tile — the
      // last tile of a portion is the one with the most keys, and it is seldom full.
      const int pos = row_valid ? start + i_row / G : 0x7fffffff;
      const int first = (row_valid && p.window > 0) ? max(0, pos - p.window + 1) : 0;
      const float sl = p.scale * kLog2e5;
      float m_ref = -INFINITY, l = 0.0f;                         // l is this thread's sum relative to m_ref
      bool ok = true;
      const int b = set;                                         // the set's S and P buffer

      for (int j = set; j < ntiles; j += 2) {
        const int use = j >> 1;
        if (!mbar_wait(&sm.s_full[b], use & 1, p.error)) { ok = false; break; }
        tc_fence_after();
        const uint32_t s_addr = tmem + lane_base + b * TK + part * CW;
        const int j0 = (t_first + j) * TK + part * CW;
        // a tile that lies wholly inside every row's visible range needs no mask (the usual case)
        const bool unmasked = __all_sync(0xffffffffu, j0 + CW - 1 <= pos && j0 >= first);
        // first pass over this thread's scores: their maximum
        float m_part = -INFINITY;
        {
          uint32_t sv[CW];
          if constexpr (CW == 64) tmem_ld64(s_addr, sv);
          else tmem_ld32(s_addr, sv);
          tmem_wait_ld();
          if (unmasked) {
            float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains instead of one
#pragma unroll
            for (int e = 0; e < CW; ++e) m4[e & 3] = fmaxf(m4[e & 3], __uint_as_float(sv[e]));
            m_part = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
          } else {
#pragma unroll
            for (int e = 0; e < CW; ++e) {
              const int key = j0 + e;
              if (key <= pos && key >= first) m_part = fmaxf(m_part, __uint_as_float(sv[e]));
            }
          }
        }
        m_part *= sl;                                            // scale > 0
        sm.xmax[set][use & 1][part][row] = m_part;
        row_group_sync<32 * SPLIT>(set, warp & 3);               // the warps of the set that share these 32 rows
        float m_tile = m_part;
#pragma unroll
        for (int o = 0; o < SPLIT; ++o) m_tile = fmaxf(m_tile, sm.xmax[set][use & 1][o][row]);
        // the reference after the tile before, which the other set has published
        float m_prev = -INFINITY;
        if (j > 0) {
          if (!mbar_wait(&sm.r_full[b ^ 1], ((j - 1) >> 1) & 1, p.error)) { ok = false; break; }
          m_prev = sm.mref[(j - 1) & 1][row];
        }
        float m_new = m_prev;
        bool grow = false;
        if (m_tile > m_prev + kRescaleThreshold || (m_prev == -INFINITY && m_tile > -INFINITY)) {
          m_new = m_tile;
          grow = true;
        }
        if (part == 0) {
          // (the slot's last reader, the other set at tile j - 1, read it before it published what was waited for above)
          sm.mref[j & 1][row] = m_new;
          __syncwarp();
          if (lane == 0) mbar_arrive(&sm.r_full[b]);
        }
        const float m_use = m_new == -INFINITY ? 0.0f : m_new;
        // this thread's sum refers to the reference of its set's last tile
        const float alpha_l = m_new == m_ref ? 1.0f : (m_ref == -INFINITY ? 0.0f : exp2f(m_ref - m_new));
        // the set's P buffer is free once the P V product of the set's last tile has finished
        if (use > 0) {
          if (!mbar_wait(&sm.p_empty[b], (use - 1) & 1, p.error)) { ok = false; break; }
        }
        // second pass, 32 scores at a time: exponentials; the probabilities go to tensor memory as packed pairs,
        // where the P V product reads them as its A operand (a masked score counts as -inf and gives 0)
        float sum = 0.0f;
#pragma unroll
        for (int c = 0; c < CW / 32; ++c) {
          uint32_t sv[32];
          tmem_ld32(s_addr + c * 32, sv);
          tmem_wait_ld();
          if (c == CW / 32 - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.s_empty[b]);          // S_b has been read: the set's next S may land
          }
          if (!unmasked) {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const int key = j0 + c * 32 + e;
              if (!(key <= pos && key >= first)) sv[e] = 0xff800000u;   // -inf
            }
          }
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(sv[2 * e]), sl, -m_use));
            const float p1 = fast_exp2(fmaf(__uint_as_float(sv[2 * e + 1]), sl, -m_use));
            sum += p0 + p1;
            __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
            pk[e] = *reinterpret_cast<uint32_t*>(&h);
          }
          tmem_st16(tmem + 384 + b * (TK / 2) + lane_base + part * (CW / 2) + c * 16, pk);
        }
        // O may only be rescaled while no P V product is running: after the product of the tile before (the other
        // set's) and before this tile's, which waits for the arrival below
        if (j > 0 && __any_sync(0xffffffffu, grow)) {
          if (!mbar_wait(&sm.p_empty[b ^ 1], ((j - 1) >> 1) & 1, p.error)) { ok = false; break; }
          tc_fence_after();
          const float alpha = m_new == m_prev ? 1.0f : (m_prev == -INFINITY ? 0.0f : exp2f(m_prev - m_new));
#pragma unroll 1
          for (int c = 0; c < OW / 32; ++c) {                    // this thread's part of the O columns
            uint32_t ov[32];
            const uint32_t o_addr = tmem_o + lane_base + part * OW + c * 32;
            tmem_ld32(o_addr, ov);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * alpha);
            tmem_st32(o_addr, ov);
          }
        }
        tmem_wait_st();
        l = l * alpha_l + sum;
        m_ref = m_new;
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.p_full[b]);
      }
      // epilogue: the row's sums, each brought to the last reference
      softmax_sync<kSoftmaxThreads>();                           // the last tile's reference is published
      {
        const float m_final = sm.mref[(ntiles - 1) & 1][row];
        sm.xsum[set * SPLIT + part][row] = (l > 0.0f && m_ref != m_final) ? l * exp2f(m_ref - m_final) : l;
      }
      softmax_sync<kSoftmaxThreads>();
      if (set == 0) {
      float l_row = 0.0f;
#pragma unroll
      for (int o = 0; o < 2 * SPLIT; ++o) l_row += sm.xsum[o][row];
      // O leaves through shared memory (the K ring is idle: every product has finished), so that the stores to
      // global memory are whole rows — 16 lanes a row — instead of 16 bytes a lane to 32 different rows, which
      // took 2.8 of a block's 59 thousand cycles per tile.
      constexpr int STAGE_STRIDE = D * 2 + 16;                   // bytes a staged row; the pad spreads rows over banks
      unsigned char* stage = sm.k[0];
      static_assert(TQ * STAGE_STRIDE <= K_STAGES * PANELS * KV_PANEL_BYTES, "the staged tile fits the K ring");
      if (ok && mbar_wait(&sm.o_ready, 0, p.error)) {
        tc_fence_after();
        const float inv = (l_row > 0.0f) ? 1.0f / l_row : 0.0f;
        if (row_valid && part == 0 && (!(l_row > 0.0f) || !isfinite(l_row))) publish_error(p.error, kAttentionDenominator);
#pragma unroll 1
        for (int c = 0; c < OW / 32; ++c) {
          uint32_t ov[32];
          tmem_ld32(tmem_o + lane_base + part * OW + c * 32, ov);
          tmem_wait_ld();
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(ov[2 * e]) * inv, __uint_as_float(ov[2 * e + 1]) * inv);
            pk[e] = *reinterpret_cast<uint32_t*>(&h);
          }
          uint4* dst = reinterpret_cast<uint4*>(stage + row * STAGE_STRIDE + (part * OW + c * 32) * 2);
#pragma unroll
          for (int e = 0; e < 4; ++e) dst[e] = make_uint4(pk[4 * e], pk[4 * e + 1], pk[4 * e + 2], pk[4 * e + 3]);
        }
      }
      first_set_sync<kSetThreads>();                             // every thread of the set, whatever its waits said
      {
        constexpr int CPR = D / 8;
        const int ch = t % CPR;
        PackedRowWalk w(tile_row0 + t / CPR, kSetThreads / CPR, G);
        for (int r_out = t / CPR; r_out < TQ && w.i < packed; r_out += kSetThreads / CPR, w.next())
          *reinterpret_cast<uint4*>(p.out + (static_cast<size_t>(row0 + w.tok) * p.heads + g * G + w.hd) * D + ch * 8) =
              *reinterpret_cast<const uint4*>(stage + r_out * STAGE_STRIDE + ch * 16);
      }
      proxy_fence();                                             // the next item's TMA boxes land where these rows lay
      }
    }
    tc_fence_before();
    __syncthreads();                                             // the item is finished everywhere
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(sm.tmem_base), "r"(512));
  }
}

}  // namespace pih

using namespace pih;

// Attention of the requests that bring more than 16 packed rows (prompt portions); rows of other requests
// are left untouched.  head_dim 64 or 128, page_size 8..64 (a power of two), kv_tensor_map from
// pih_make_kv_tensor_map.  rows: the rows of the step (of q); tile_max_q: the most rows of such a request — the two
// bound the grid, which rows are whose is read from cu_q on the device.  PIH_ERR_UNSUPPORTED otherwise.
extern "C" int pih_attention_prefill_tcgen05(const void* q, int q_stride, int rows, void* out, const int* block_table,
                                             int table_width, const int* cu_q, const int* q_start, int num_requests,
                                             int tile_max_q, int heads, int kv_heads, int head_dim, int page_size,
                                             int num_pages, float scale, int window, const void* kv_tensor_map,
                                             uint32_t* error, void* stream) {
  if (tile_max_q <= 0) return 0;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || num_requests <= 0 || rows <= 0 ||
      kv_heads > 65535 || q_stride % 8 || window < 0 || table_width <= 0)
    return PIH_ERR_BAD_ARGUMENT;
  int shift = -1;
  for (int s = 3; s <= 6; ++s)
    if ((1 << s) == page_size) shift = s;
  if (shift < 0 || kv_tensor_map == nullptr || (head_dim != 64 && head_dim != 128)) return PIH_ERR_UNSUPPORTED;
  PrefillParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.q_stride = q_stride;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.block_table = block_table;
  p.table_width = table_width;
  p.cu_q = cu_q;
  p.q_start = q_start;
  p.heads = heads;
  p.kv_heads = kv_heads;
  p.page_size = page_size;
  p.page_shift = shift;
  p.num_pages = num_pages;
  p.num_requests = num_requests;
  p.scale = scale;
  p.window = window;
  p.error = error;
  CUtensorMap map;
  memcpy(&map, kv_tensor_map, sizeof(CUtensorMap));
  const int G = heads / kv_heads;
  // row tiles of all requests together: no more than the step's packed rows hold, one partial tile a request
  // more; and no more than every request at its longest
  const long long by_rows = (static_cast<long long>(rows) * G + TQ - 1) / TQ + num_requests;
  const long long by_requests = static_cast<long long>(num_requests) * ((tile_max_q * G + TQ - 1) / TQ);
  const long long tiles = by_rows < by_requests ? by_rows : by_requests;
  if (tiles > 0x7fffffffLL) return PIH_ERR_BAD_ARGUMENT;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  p.pair_above = sms;                  // single tiles while every tile finds an SM of its own; beyond that, pairs
                                       // (a 2048-token prompt: 256 single tiles in two uneven waves 40 us, 128 pairs 31 us)
  dim3 grid(static_cast<unsigned>(tiles), kv_heads, 1);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  static bool configured[2] = {false, false};
  if (head_dim == 128) {
    // two threads per row; four (sixteen softmax warps) were measured no faster once the MMA issue was off the
    // critical path: the exponentials are bound by the special-function unit, not by latency
    constexpr int SPLIT = 2;
    const int smem = static_cast<int>(sizeof(PrefillSmem<128, SPLIT>)) + 1024;
    if (!configured[0]) {
      cudaError_t e = cudaFuncSetAttribute(attn_prefill_tcgen05_kernel<128, SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return static_cast<int>(e);
      configured[0] = true;
    }
    launch_kernel(attn_prefill_tcgen05_kernel<128, SPLIT>, dim3(grid), dim3(256 * SPLIT + 128), smem, s, p, map);
  } else {
    const int smem = static_cast<int>(sizeof(PrefillSmem<64, 2>)) + 1024;
    if (!configured[1]) {
      cudaError_t e = cudaFuncSetAttribute(attn_prefill_tcgen05_kernel<64, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return static_cast<int>(e);
      configured[1] = true;
    }
    launch_kernel(attn_prefill_tcgen05_kernel<64, 2>, dim3(grid), dim3(640), smem, s, p, map);
  }
  PIH_LAUNCH_CHECK();
  return 0;
}
