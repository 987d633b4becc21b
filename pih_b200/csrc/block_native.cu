// One call per block: the kernels of a pre-norm block with paged attention and a SwiGLU feed-forward, issued from
// native code.
//
// The parts (pih_b200/parts) put a block together from single ops, each a call through the binding layer: five to
// nine calls a layer, about 20 us of host time each.  A step that is replayed from a CUDA graph does not notice; a
// step that is not — a prompt portion of a length not seen before, a batch whose make-up has just changed — is
// bound by exactly this host time.  This file issues the same kernels, in the same order and with the same
// choices, from one call: the reference's engine likewise runs a layer from C++
// (plugins/model-qwen3/qwen3_bf16_execution_schedule.cpp:19-39 is the order; nvidia_qwen3_bf16_engine.cpp issues it).
//
//   h' = h + delta; qkv = norm_in(h') . Wqkv^T            few rows: one kernel; else add + norm, then the library product
//   q/k norm, rotation, cache append, attention           decode steps: one kernel; else the q/k kernel, then attention
//   h'' = h' + attn . Wo^T                                few rows: the add rides in the product's epilogue
//   act = SwiGLU(norm_post(h'') . Wgu^T)                  few rows: one kernel; else add + norm, product, SiLU-mul
//   h''' = h'' + act . Wd^T                               as the output projection
//
// Products of more than `skinny_max_rows` rows in bfloat16 go to cuBLAS, as they do through torch on the other path
// and as the reference's go to cuBLASLt (src/backend/cuda/gemm_plan.cpp:192-197); in float32 every product runs on
// the pack's own FMA kernel.  cuBLAS is looked up in the library that the process has already loaded.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <stdint.h>
#include <stdio.h>

#include "common.cuh"

extern "C" {
int pih_rmsnorm(int dtype, int weight_dtype, void* x, const void* delta, const void* weight, void* out, const int* rows,
                int out_rows, int width, float eps, void* stream);
int pih_qk_norm_rope_kv_write(int dtype, int weight_dtype, void* qkv, int row_stride, int rows, int heads, int kv_heads,
                              int head_dim, const void* q_w, const void* k_w, float eps, const float* rope,
                              int rotary_dim, int max_pos, const int* positions, const int* slot_mapping, void* cache,
                              int page_size, int num_pages, int write_kv, uint32_t* error, void* stream);
int pih_silu_mul(int dtype, const void* gate_up, void* out, long long rows, int inter, int interleave, void* stream);
int pih_gemm_simt(int in_dtype, int out_dtype, const void* A, const void* W, void* C, int M, int N, int K, long long lda,
                  long long ldw, long long ldc, void* stream);
int pih_pair_swiglu_wanted(int rows, int n);
int pih_gemm_tcgen05_pair(int out_dtype, const void* A, const void* W, void* C, int M, int N, int K, long long lda,
                          long long ldw, long long ldc, int tile_n, int swiglu, uint32_t* error, void* stream);
int pih_gemm_skinny(const void* x, const void* delta, void* x_out, int norm_dtype, const void* norm_w, float eps,
                    const void* W, void* out, const void* residual, int M, int N, int K, long long ldx, long long ldw,
                    long long ldo, int swiglu, uint32_t* error, void* stream);
int pih_paged_attention_generic(int dtype, const void* q, int q_stride, void* out, const void* cache,
                                const int* block_table, int table_width, const int* request_of_row, const int* positions,
                                int rows, int heads, int kv_heads, int head_dim, int page_size, int num_pages, float scale,
                                int window, uint32_t* error, void* stream);
int pih_paged_attention_mma(const void* q, int q_stride, void* out, const void* cache, const int* block_table,
                            int table_width, const int* cu_q, const int* q_start, int rows, int num_requests,
                            int tile_max_q, int dec_tok_cap, int dec_max_ctx, int heads, int kv_heads, int head_dim,
                            int page_size, int num_pages, float scale, int window, int split, int max_splits,
                            const int* max_ctx_ptr, float* scratch, const void* kv_tensor_map, uint32_t* error,
                            void* stream);
int pih_qk_attention_fused(const void* qkv, int q_stride, void* out, void* cache, const int* block_table, int table_width,
                           const int* cu_q, const int* q_start, int rows, int num_requests, int dec_tok_cap,
                           int dec_max_ctx, int heads, int kv_heads, int head_dim, int page_size, int num_pages,
                           float scale, int window, int split, int max_splits, const int* max_ctx_ptr, float* scratch,
                           const void* kv_tensor_map, int norm_dtype, const void* q_norm_w, const void* k_norm_w,
                           float eps, const float* rope, int max_pos, int write_kv, uint32_t* error, void* stream);
int pih_attention_prefill_tcgen05(const void* q, int q_stride, int rows, void* out, const int* block_table, int table_width,
                                  const int* cu_q, const int* q_start, int num_requests, int tile_max_q, int heads,
                                  int kv_heads, int head_dim, int page_size, int num_pages, float scale, int window,
                                  const void* kv_tensor_map, uint32_t* error, void* stream);
}

// ---- what Python hands over (mirrored field by field in pih_b200/kernels/native_block.py) ---------------------------

struct PihStepArgs {                     // the same for every block of a step
  int dtype;                             // PIH_F32 or PIH_BF16
  int rows, num_requests;
  int skinny_max_rows, fused_residual;
  const int* positions;
  const int* request_of_row;
  const int* cu_q;
  const int* q_start;
  const int* max_ctx_ptr;                // nullable
  uint32_t* error;
  void* stream;
  void* library_workspace;               // for the library's products; allocated by the caller, capture-safe
  long long library_workspace_bytes;
};

struct PihAttentionArgs {                // per step, cache group and attention geometry
  const int* block_table;
  const int* slot_mapping;
  int table_width, page_size, num_pages;
  int tensor_cores;                      // 0: the generic kernel
  int try_fused;                         // a decode step: the attention kernel may do the q/k work itself
  int tcgen05_prefill;                   // prompt portions on the tcgen05 kernel
  int tma_split;                         // the split kernel takes the cache's tensor map
  int tile_max_q, dec_cap, dec_ctx, split, nsplits;
  float* scratch;
};

struct PihBlockArgs {
  // weights and constants
  const void* norm_in_w;
  const void* norm_post_w;
  const void* w_qkv;
  const void* w_o;
  const void* w_gate_up;
  const void* w_down;
  const void* q_norm_w;                  // nullable
  const void* k_norm_w;
  const float* rope;                     // nullable
  long long ld_qkv, ld_o, ld_gate_up, ld_down;
  int norm_w_dtype, qk_norm_dtype;
  float norm_in_eps, norm_post_eps, qk_eps, scale;
  int hidden, heads, kv_heads, head_dim, intermediate, interleave, window, rotary_dim, max_pos;
  int qkv_cols;                          // heads * head_dim (+ 2 kv_heads * head_dim when the entry writes its cache)
  // this schedule entry's cache
  void* kv_cache;
  const void* kv_map;                    // nullable
  int writable;
  // activations
  void* h;                               // [rows, hidden]
  const void* delta;                     // nullable
  void* h_sum;                           // workspaces, each [rows, ...]
  void* h_sum2;
  void* xn;
  void* qkv;
  void* attn;
  void* o;
  void* h2;
  void* gate_up;
  void* act;
  void* y;
  void* h3;
  // result: which buffers hold the stream and what is still to be added to it
  int out_h;                             // 0 h, 1 h_sum, 2 h2, 3 h3, 4 h_sum2
  int out_delta;                         // 0 none, 1 o, 2 y
  int launched;                          // kernels (and library products) that this call queued
};

namespace {

// ---- the library product, looked up at run time ---------------------------------------------------------------------
typedef int (*CreateFn)(void**);
typedef int (*SetStreamFn)(void*, cudaStream_t);
typedef int (*SetWorkspaceFn)(void*, void*, size_t);
typedef int (*SetMathFn)(void*, int);
typedef int (*GemmExFn)(void*, int, int, int, int, int, const void*, const void*, int, int, const void*, int, int,
                        const void*, void*, int, int, int, int);
struct Library {
  void* handle = nullptr;
  SetStreamFn set_stream = nullptr;
  SetWorkspaceFn set_workspace = nullptr;
  GemmExFn gemm = nullptr;
  int state = 0;                         // 0 not tried, 1 ready, -1 unavailable
};
Library g_lib[64];

Library* library() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  Library& L = g_lib[dev];
  if (L.state == 0) {
    L.state = -1;
    void* so = dlopen("libcublas.so.12", RTLD_NOW | RTLD_NOLOAD);
    if (so == nullptr) so = dlopen("libcublas.so.12", RTLD_NOW);
    if (so == nullptr) so = dlopen("libcublas.so", RTLD_NOW);
    if (so != nullptr) {
      CreateFn create = reinterpret_cast<CreateFn>(dlsym(so, "cublasCreate_v2"));
      SetMathFn set_math = reinterpret_cast<SetMathFn>(dlsym(so, "cublasSetMathMode"));
      L.set_stream = reinterpret_cast<SetStreamFn>(dlsym(so, "cublasSetStream_v2"));
      L.set_workspace = reinterpret_cast<SetWorkspaceFn>(dlsym(so, "cublasSetWorkspace_v2"));
      L.gemm = reinterpret_cast<GemmExFn>(dlsym(so, "cublasGemmEx"));
      if (create && set_math && L.set_stream && L.set_workspace && L.gemm && create(&L.handle) == 0) {
        // sums in 32-bit all the way: no reduced-precision partial sums in split-k reductions (CUBLAS_DEFAULT_MATH |
        // CUBLAS_MATH_DISALLOW_REDUCED_PRECISION_REDUCTION)
        set_math(L.handle, 0 | 16);
        L.state = 1;
      }
    }
  }
  return L.state == 1 ? &L : nullptr;
}

// out[M, N] = x[M, K] . w[N, K]^T, rows of x, w and out `ldx`, `ldw`, `ldo` elements apart
int product(const PihStepArgs& s, const void* x, long long ldx, const void* w, long long ldw, void* out, long long ldo,
            int M, int N, int K) {
  if (M <= 0 || N <= 0) return 0;
  if (s.dtype == PIH_F32) return pih_gemm_simt(PIH_F32, PIH_F32, x, w, out, M, N, K, ldx, ldw, ldo, s.stream);
  Library* L = library();
  if (L == nullptr) return PIH_ERR_UNSUPPORTED;
  if (L->set_stream(L->handle, static_cast<cudaStream_t>(s.stream)) != 0) return PIH_ERR_UNSUPPORTED;
  if (L->set_workspace(L->handle, s.library_workspace, static_cast<size_t>(s.library_workspace_bytes)) != 0)
    return PIH_ERR_UNSUPPORTED;
  const float one = 1.0f, zero = 0.0f;
  // row-major out = x . w^T is column-major out^T [N, M] = w [K, N]^T . x [K, M]
  const int CUBLAS_OP_N = 0, CUBLAS_OP_T = 1, CUDA_R_16BF = 14, CUBLAS_COMPUTE_32F = 68, CUBLAS_GEMM_DEFAULT = -1;
  const int rc = L->gemm(L->handle, CUBLAS_OP_T, CUBLAS_OP_N, N, M, K, &one, w, CUDA_R_16BF, static_cast<int>(ldw), x,
                         CUDA_R_16BF, static_cast<int>(ldx), &zero, out, CUDA_R_16BF, static_cast<int>(ldo),
                         CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
  return rc == 0 ? 0 : 1000 + rc;
}

// A second stream with the two events of a fork and a join, one set a device, made at the first use (which is not
// inside a graph capture: a step of a new shape runs uncaptured first).
struct Fork {
  cudaStream_t stream = nullptr;
  cudaEvent_t forked = nullptr, joined = nullptr;
  int state = 0;                         // 0 not tried, 1 ready, -1 unavailable
};
Fork g_fork[64];
int g_attention_side_by_side = 1;

Fork* side_stream() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  Fork& f = g_fork[dev];
  if (f.state == 0) {
    f.state = -1;
    if (cudaStreamCreateWithFlags(&f.stream, cudaStreamNonBlocking) == cudaSuccess &&
        cudaEventCreateWithFlags(&f.forked, cudaEventDisableTiming) == cudaSuccess &&
        cudaEventCreateWithFlags(&f.joined, cudaEventDisableTiming) == cudaSuccess)
      f.state = 1;
  }
  return f.state == 1 ? &f : nullptr;
}

bool few_rows(const PihStepArgs& s) { return s.dtype == PIH_BF16 && s.rows <= s.skinny_max_rows && s.rows <= 16; }

#define PIH_TRY(call)            \
  do {                           \
    const int rc_ = (call);      \
    if (rc_ != 0) return rc_;    \
    ++b->launched;               \
  } while (0)

}  // namespace

// 1 (the default): in a step with prompt portions and decoding requests the two attention kernels run side by side;
// 0: one after the other in the step's stream.  Returns the previous setting.
extern "C" int pih_set_attention_side_by_side(int on) {
  const int before = g_attention_side_by_side;
  g_attention_side_by_side = on ? 1 : 0;
  return before;
}

// Returns 0, or the first failing kernel's code (PIH_ERR_* or a cudaError_t; 1000 + n: the library product failed
// with status n), with whatever was launched before it left queued.
extern "C" int pih_prenorm_attention_swiglu_block(const PihStepArgs* sp, const PihAttentionArgs* ap, PihBlockArgs* b) {
  const PihStepArgs& s = *sp;
  const PihAttentionArgs& a = *ap;
  const int T = s.rows, H = b->hidden, D = b->head_dim;
  const int q_size = b->heads * D;
  void* h = b->h;
  const void* delta = b->delta;
  b->out_h = 0;
  b->launched = 0;

  // ---- q/k/v product with the add and the norm in front
  bool done = false;
  if (few_rows(s)) {
    const int rc = pih_gemm_skinny(h, delta, b->h_sum, b->norm_w_dtype, b->norm_in_w, b->norm_in_eps, b->w_qkv, b->qkv,
                                   nullptr, T, b->qkv_cols, H, H, b->ld_qkv, b->qkv_cols, 0, s.error, s.stream);
    if (rc == 0) {
      done = true;
      ++b->launched;
      if (delta != nullptr) {
        h = b->h_sum;
        b->out_h = 1;
      }
    } else if (rc != PIH_ERR_UNSUPPORTED) {
      return rc;
    }
  }
  if (!done) {
    PIH_TRY(pih_rmsnorm(s.dtype, b->norm_w_dtype, h, delta, b->norm_in_w, b->xn, nullptr, T, H, b->norm_in_eps, s.stream));
    PIH_TRY(product(s, b->xn, H, b->w_qkv, b->ld_qkv, b->qkv, b->qkv_cols, T, b->qkv_cols, H));
  }

  // ---- q/k norm, rotation, cache append, attention
  done = false;
  if (a.try_fused && (b->rope == nullptr || b->rotary_dim == D)) {
    const int rc = pih_qk_attention_fused(b->qkv, b->qkv_cols, b->attn, b->kv_cache, a.block_table, a.table_width, s.cu_q,
                                          s.q_start, T, s.num_requests, a.dec_cap, a.dec_ctx, b->heads, b->kv_heads, D,
                                          a.page_size, a.num_pages, b->scale, b->window, a.split, a.nsplits,
                                          s.max_ctx_ptr, a.scratch, b->kv_map, b->qk_norm_dtype, b->q_norm_w, b->k_norm_w,
                                          b->qk_eps, b->rope, b->rope != nullptr ? b->max_pos : 0, b->writable, s.error,
                                          s.stream);
    if (rc == 0) {
      done = true;
      ++b->launched;
    } else if (rc != PIH_ERR_UNSUPPORTED) {
      return rc;
    }
  }
  if (!done) {
    PIH_TRY(pih_qk_norm_rope_kv_write(s.dtype, b->q_norm_w != nullptr ? b->qk_norm_dtype : s.dtype, b->qkv, b->qkv_cols, T,
                                      b->heads, b->kv_heads, D, b->q_norm_w, b->k_norm_w, b->qk_eps, b->rope,
                                      b->rotary_dim, b->rope != nullptr ? b->max_pos : 0, s.positions, a.slot_mapping,
                                      b->kv_cache, a.page_size, a.num_pages, b->writable, s.error, s.stream));
    if (a.tensor_cores) {
      int tile_max_q = a.tile_max_q;
      if (tile_max_q > 0 && a.tcgen05_prefill && b->kv_map != nullptr) {
        if (a.dec_cap > 0 && g_attention_side_by_side) {       // the fork for the decoding requests' kernel (below)
          Fork* fork = side_stream();
          if (fork != nullptr) {
            const cudaError_t e = cudaEventRecord(fork->forked, static_cast<cudaStream_t>(s.stream));
            if (e != cudaSuccess) return static_cast<int>(e);
          }
        }
        PIH_TRY(pih_attention_prefill_tcgen05(b->qkv, b->qkv_cols, T, b->attn, a.block_table, a.table_width, s.cu_q, s.q_start,
                                              s.num_requests, tile_max_q, b->heads, b->kv_heads, D, a.page_size,
                                              a.num_pages, b->scale, b->window, b->kv_map, s.error, s.stream));
        tile_max_q = 0;
      }
      if (tile_max_q > 0 || a.dec_cap > 0) {
        // A mixed step's decoding requests are other requests than its prompt portions, and their kernel other SMs'
        // work (a block of the prompt kernel fills an SM's shared memory): it runs beside the prompt kernel, in a
        // stream that forks from this one behind the q/k kernel and joins it again before the output projection.
        Fork* fork = (a.tile_max_q > 0 && tile_max_q == 0 && a.dec_cap > 0 && g_attention_side_by_side) ? side_stream() : nullptr;
        void* stream = s.stream;
        if (fork != nullptr) {
          const cudaError_t e = cudaStreamWaitEvent(fork->stream, fork->forked, 0);
          if (e != cudaSuccess) return static_cast<int>(e);
          stream = fork->stream;
        }
        PIH_TRY(pih_paged_attention_mma(b->qkv, b->qkv_cols, b->attn, b->kv_cache, a.block_table, a.table_width, s.cu_q,
                                        s.q_start, T, s.num_requests, tile_max_q, a.dec_cap, a.dec_ctx, b->heads,
                                        b->kv_heads, D, a.page_size, a.num_pages, b->scale, b->window, a.split, a.nsplits,
                                        s.max_ctx_ptr, a.dec_cap > 0 ? a.scratch : nullptr,
                                        (a.tma_split && a.dec_cap > 0) ? b->kv_map : nullptr, s.error, stream));
        if (fork != nullptr) {
          cudaError_t e = cudaEventRecord(fork->joined, fork->stream);
          if (e == cudaSuccess) e = cudaStreamWaitEvent(static_cast<cudaStream_t>(s.stream), fork->joined, 0);
          if (e != cudaSuccess) return static_cast<int>(e);
        }
      }
    } else {
      PIH_TRY(pih_paged_attention_generic(s.dtype, b->qkv, b->qkv_cols, b->attn, b->kv_cache, a.block_table, a.table_width,
                                          s.request_of_row, s.positions, T, b->heads, b->kv_heads, D, a.page_size,
                                          a.num_pages, b->scale, b->window, s.error, s.stream));
    }
  }

  // ---- output projection, the residual add in its epilogue for few rows
  const void* pending = nullptr;         // what is still to be added to the stream
  done = false;
  if (few_rows(s) && s.fused_residual) {
    const int rc = pih_gemm_skinny(b->attn, nullptr, nullptr, 0, nullptr, 0.0f, b->w_o, b->h2, h, T, H, q_size, q_size,
                                   b->ld_o, H, 0, s.error, s.stream);
    if (rc == 0) {
      done = true;
      ++b->launched;
      h = b->h2;
      b->out_h = 2;
    } else if (rc != PIH_ERR_UNSUPPORTED) {
      return rc;
    }
  }
  if (!done) {
    int rc = PIH_ERR_UNSUPPORTED;
    if (few_rows(s))
      rc = pih_gemm_skinny(b->attn, nullptr, nullptr, 0, nullptr, 0.0f, b->w_o, b->o, nullptr, T, H, q_size, q_size, b->ld_o,
                           H, 0, s.error, s.stream);
    if (rc == PIH_ERR_UNSUPPORTED) rc = product(s, b->attn, q_size, b->w_o, b->ld_o, b->o, H, T, H, q_size);
    if (rc != 0) return rc;
    ++b->launched;
    pending = b->o;
  }

  // ---- gate/up product with the add and the norm in front and SiLU-mul behind
  const int I = b->intermediate;
  done = false;
  if (few_rows(s) && b->interleave == 8) {
    const int rc = pih_gemm_skinny(h, pending, b->h_sum2, b->norm_w_dtype, b->norm_post_w, b->norm_post_eps, b->w_gate_up,
                                   b->act, nullptr, T, 2 * I, H, H, b->ld_gate_up, I, 1, s.error, s.stream);
    if (rc == 0) {
      done = true;
      ++b->launched;
      if (pending != nullptr) {
        h = b->h_sum2;
        b->out_h = 4;
      }
    } else if (rc != PIH_ERR_UNSUPPORTED) {
      return rc;
    }
  }
  if (!done) {
    PIH_TRY(pih_rmsnorm(s.dtype, b->norm_w_dtype, h, pending, b->norm_post_w, b->xn, nullptr, T, H, b->norm_post_eps,
                        s.stream));
    // many rows: the pack's own product on pairs of SMs, SiLU-mul in its epilogue (the [T, 2 I] product never
    // reaches memory); else the library's product and the separate kernel
    if (s.dtype == PIH_BF16 && b->interleave == 8 && pih_pair_swiglu_wanted(T, 2 * I)) {
      const int rc = pih_gemm_tcgen05_pair(PIH_BF16, b->xn, b->w_gate_up, b->act, T, 2 * I, H, H, b->ld_gate_up, I, 0, 1,
                                           s.error, s.stream);
      if (rc == 0) {
        done = true;
        ++b->launched;
      } else if (rc != PIH_ERR_UNSUPPORTED) {
        return rc;
      }
    }
  }
  if (!done) {
    PIH_TRY(product(s, b->xn, H, b->w_gate_up, b->ld_gate_up, b->gate_up, 2 * I, T, 2 * I, H));
    PIH_TRY(pih_silu_mul(s.dtype, b->gate_up, b->act, T, I, b->interleave, s.stream));
  }

  // ---- down product, the residual add in its epilogue for few rows
  b->out_delta = 0;
  if (few_rows(s) && s.fused_residual) {
    const int rc = pih_gemm_skinny(b->act, nullptr, nullptr, 0, nullptr, 0.0f, b->w_down, b->h3, h, T, H, I, I, b->ld_down,
                                   H, 0, s.error, s.stream);
    if (rc == 0) {
      ++b->launched;
      b->out_h = 3;
      return 0;
    }
    if (rc != PIH_ERR_UNSUPPORTED) return rc;
  }
  int rc = PIH_ERR_UNSUPPORTED;
  if (few_rows(s))
    rc = pih_gemm_skinny(b->act, nullptr, nullptr, 0, nullptr, 0.0f, b->w_down, b->y, nullptr, T, H, I, I, b->ld_down, H, 0,
                         s.error, s.stream);
  if (rc == PIH_ERR_UNSUPPORTED) rc = product(s, b->act, I, b->w_down, b->ld_down, b->y, H, T, H, I);
  if (rc != 0) return rc;
  ++b->launched;
  b->out_delta = 2;
  return 0;
}
