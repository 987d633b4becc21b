"""``CudaOps``: the calls that parts make, bound to the kernel pack through ctypes.

Every method launches hand-written kernels from ``csrc/`` on the current
CUDA stream.  Matrix products in bfloat16 go to the library (cuBLAS through
``torch.mm``) where the reference does the same
(src/backend/cuda/gemm_plan.cpp:192-197 runs every product through
cuBLASLt); in float32 they run on the pack's own FMA kernel so that no
reduced-precision mode can slip in.  Nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build

_DT = {torch.float32: 0, torch.bfloat16: 1}
_ERRORS = {1: "a token id is outside the vocabulary", 2: "a row maps to no cache page",
           3: "logits contain a non-finite value", 4: "a position is outside the rotation table",
           5: "attention softmax denominator is not positive and finite", 6: "a device wait timed out"}

c_void_p, c_int, c_float, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(0 if t is None else t.data_ptr())


class KernelError(RuntimeError):
    pass


def error_text(code: int) -> str:
    """What a value of the device's error word means."""
    return _ERRORS.get(code, f"error code {code}")


class CudaOps:
    def __init__(self, device=None):
        if not torch.cuda.is_available():
            raise RuntimeError("pih_b200 runs on a CUDA device only (there is no CPU path), "
                               "and torch.cuda.is_available() is False")
        self.device = torch.device(device if device is not None else "cuda:0")
        if self.device.type != "cuda":
            raise RuntimeError(f"pih_b200 runs on a CUDA device only, got {self.device}")
        major, minor = torch.cuda.get_device_capability(self.device)
        if major != 10:
            raise RuntimeError(f"the kernel pack is built for sm_100a; this device is sm_{major}{minor}")
        path = build.library_path()
        try:
            self.lib = ctypes.CDLL(path)
        except OSError as e:
            raise RuntimeError(f"pih_b200: the kernel pack {path} could not be loaded: {e}") from None
        self.library_path = path
        # library products must accumulate in 32-bit all the way: no bf16 partial sums in split-K
        # reductions, no TF32
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        torch.backends.cuda.matmul.allow_tf32 = False
        self._device_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self._error = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.launches = 0
        self._attn_scratch = None          # partials of the split-KV attention kernel, grown on demand
        self._retired_scratch = []
        self._kv_maps = {}                 # cache tensor (address, shape) -> 128-byte TMA descriptor
        self.tma_attention = True          # False: the split kernel gathers with cp.async instead of TMA
        self.tcgen05_attention = True      # False: prompt portions use the mma.sync tile kernel
        self.fused_qk_attention = True     # decode-only steps: q/k norm, rotation and cache append inside the attention kernel
        self.fused_qk_max_requests = 32    # ... up to this batch (measured: 16 requests +4 %, 32 even, 64 -1.6 %)
        self.cluster_attention = True      # False: splits always merge through scratch memory and tickets
        self.attention_split = 0           # keys per split of the decode attention kernel; 0: from the context, on the device
        self.tensor_core_attention = True  # False: bf16 attention runs on the generic kernel too
        self._tcgen05_swiglu_min_rows = 1536     # the library's default (see the property)
        self.tcgen05_min_rows = None       # bf16 products with at least this many rows use the pack's tcgen05 kernel
        self.skinny_max_rows = 16          # bf16 products with at most this many rows use the fused few-rows kernel
        self.fused_residual = True         # ... and add the residual in the epilogue of output projections
        self.native_blocks = True          # blocks of the built-in parts are issued by one native call each
        self._native = None
        self._declare()

    @property
    def tcgen05_swiglu_min_rows(self):
        """Prompt portions of at least this many rows run their gate/up product on the pack's tcgen05 kernel on
        pairs of SMs with SiLU-mul in its epilogue, when its tiles fill the SM pairs well (see
        pih_pair_swiglu_wanted); None: never.  The setting is the library's: native blocks follow it."""
        return self._tcgen05_swiglu_min_rows

    @tcgen05_swiglu_min_rows.setter
    def tcgen05_swiglu_min_rows(self, rows) -> None:
        self.set_pair_swiglu_rule(rows)

    def set_pair_swiglu_rule(self, min_rows, min_fill_percent: int = -1) -> None:
        """``min_rows`` as ``tcgen05_swiglu_min_rows``; ``min_fill_percent``: how full the tiles must make the
        rounds of SM pairs (80 by default; 0 sends every shape of enough rows to that kernel; -1: unchanged)."""
        self._tcgen05_swiglu_min_rows = min_rows
        self.lib.pih_set_pair_swiglu_rule(int(min_rows) if min_rows else 0, int(min_fill_percent))

    # -- plumbing ---------------------------------------------------------------
    def _declare(self) -> None:
        lib = self.lib
        for name in ("pih_embedding", "pih_rmsnorm", "pih_qk_norm_rope_kv_write", "pih_silu_mul",
                     "pih_gather_rows", "pih_gemm_simt", "pih_paged_attention_generic", "pih_argmax",
                     "pih_sample", "pih_selected_logprob", "pih_top_logprobs", "pih_paged_attention_mma", "pih_gemm_tcgen05", "pih_make_kv_tensor_map",
                     "pih_attention_prefill_tcgen05", "pih_gemm_skinny", "pih_set_dependent_launch", "pih_set_attention_cluster_merge",
                     "pih_gemm_skinny_f32out",
                     "pih_qk_attention_fused", "pih_gemm_tcgen05_pair", "pih_set_attention_side_by_side", "pih_set_skinny_rule"):
            getattr(lib, name).restype = c_int
        lib.pih_attention_scratch_floats.restype = c_ll
        lib.pih_top_logprobs_scratch_words.restype = c_ll

    def _native_supports(self, block) -> bool:
        from .native_block import NativeBlocks
        return NativeBlocks.supports(block)

    def native_block(self, block, h, delta, step, cache):
        """A pre-norm block of the built-in parts through one native call (``native_block.NativeBlocks``); None when
        that path is off or does not take the block."""
        if not self.native_blocks:
            return None
        if self._native is None:
            from .native_block import NativeBlocks
            self._native = NativeBlocks(self)
        return self._native.run(block, h, delta, step, cache)

    def set_dependent_launch(self, on: bool) -> bool:
        """Whether the pack's kernels are launched so that each may begin while the one before it drains
        (programmatic dependent launch; the default).  Returns the previous setting.  The setting is the
        library's, not this object's; CUDA graphs keep the setting they were captured under."""
        return bool(self.lib.pih_set_dependent_launch(1 if on else 0))

    def set_skinny_rule(self, on: bool) -> bool:
        """Whether the few-rows product declines the shapes for which the library's product with the separate
        kernels is faster (the default) or takes every shape it can.  Returns the previous setting (the library's)."""
        return bool(self.lib.pih_set_skinny_rule(1 if on else 0))

    def set_attention_side_by_side(self, on: bool) -> bool:
        """Whether, in a step with prompt portions and decoding requests, native blocks run the two attention
        kernels side by side — the decoding requests' in a stream that forks behind the q/k kernel and joins before
        the output projection (the default) — or one after the other.  Returns the previous setting; the setting is
        the library's, and CUDA graphs keep the one they were captured under."""
        return bool(self.lib.pih_set_attention_side_by_side(1 if on else 0))

    def set_attention_cluster_merge(self, on):
        """Whether 2 to 8 splits of one (request, kv head) of the decode attention run as a thread-block
        cluster that merges through distributed shared memory (True, the default: small partials are sent to
        the block that finishes them, larger ones fetched by it; "fetched": always fetched) or through scratch
        memory and tickets (False).  Returns the previous setting; the setting is the library's."""
        self.cluster_attention = bool(on)
        before = self.lib.pih_set_attention_cluster_merge(2 if on == "fetched" else 1 if on else 0)
        return "fetched" if before == 2 else bool(before)

    def _stream(self):
        # the raw handle of the current stream (torch.cuda.current_stream builds a Stream object: 8 us a call,
        # four milliseconds over the launches of an uncaptured step)
        return c_void_p(torch._C._cuda_getCurrentRawStream(self._device_index))

    def _check(self, rc: int, what: str) -> None:
        self.launches += 1
        if rc == 0:
            return
        if rc == -1:
            raise KernelError(f"{what}: bad argument")
        if rc == -2:
            raise KernelError(f"{what}: this size is not supported by the kernel")
        raise KernelError(f"{what}: CUDA error {rc}")

    @property
    def error_word(self) -> torch.Tensor:
        """int32 [1] on the device: 0, or the code of the first fault that a kernel reported since it was cleared."""
        return self._error

    def clear_errors(self) -> None:
        """Zero the error word (queued on the current stream, behind the kernels already queued there)."""
        self._error.zero_()

    def check_errors(self) -> None:
        """Read the device error word (synchronises); raise if a kernel reported something."""
        code = int(self._error.item())
        if code:
            self.clear_errors()
            raise KernelError(f"a kernel reported: {error_text(code)}")

    def _err(self):
        return c_void_p(self._error.data_ptr())

    # -- ops ----------------------------------------------------------------------
    def embedding(self, table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        rows, (vocab, hidden) = ids.shape[0], table.shape
        out = torch.empty(rows, hidden, dtype=table.dtype, device=table.device)
        rc = self.lib.pih_embedding(_DT[table.dtype], _ptr(table), _ptr(ids), _ptr(out), rows, hidden, vocab,
                                    self._err(), self._stream())
        self._check(rc, "embedding")
        return out

    def rmsnorm(self, x: torch.Tensor, weight: torch.Tensor, eps: float, delta: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        width = x.shape[-1]
        assert x.is_contiguous() and (delta is None or (delta.is_contiguous() and delta.shape == x.shape))
        n_out = x.numel() // width if rows is None else rows.shape[0]
        out = torch.empty((n_out, width) if rows is not None else x.shape, dtype=x.dtype, device=x.device)
        rc = self.lib.pih_rmsnorm(_DT[x.dtype], _DT[weight.dtype], _ptr(x), _ptr(delta), _ptr(weight), _ptr(out),
                                  _ptr(rows), n_out, width, c_float(eps), self._stream())
        self._check(rc, "rmsnorm")
        return out

    def linear(self, x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """``x [M,K] . w [N,K]^T -> [M,N]``; fp32 accumulation; the output is
        rounded once to ``out_dtype`` (default: the dtype of ``x``)."""
        M, K = x.shape
        N = w.shape[0]
        out_dtype = out_dtype or x.dtype
        assert w.shape[1] == K and x.dtype == w.dtype and x.stride(1) == 1 and w.stride(1) == 1
        if x.dtype == torch.float32:
            out = torch.empty(M, N, dtype=torch.float32, device=x.device)
            rc = self.lib.pih_gemm_simt(0, 0, _ptr(x), _ptr(w), _ptr(out), M, N, K, c_ll(x.stride(0)),
                                        c_ll(w.stride(0)), c_ll(N), self._stream())
            self._check(rc, "gemm_simt")
            return out
        if out_dtype == torch.bfloat16 and M <= self.skinny_max_rows:
            out = self.linear_skinny(x, w)
            if out is not None:
                return out
        if out_dtype == torch.float32 and M <= self.skinny_max_rows and K % 32 == 0:
            out = torch.empty(M, N, dtype=torch.float32, device=x.device)
            rc = self.lib.pih_gemm_skinny_f32out(_ptr(x), _ptr(w), _ptr(out), M, N, K, c_ll(x.stride(0)),
                                                 c_ll(w.stride(0)), c_ll(N), self._err(), self._stream())
            if rc != -2:
                self._check(rc, "gemm_skinny_f32out")
                return out
        if self.tcgen05_min_rows is not None and M >= self.tcgen05_min_rows:
            out = self.linear_tcgen05(x, w, out_dtype)
            if out is not None:
                return out
        if out_dtype == torch.float32:
            return torch.mm(x, w.t(), out_dtype=torch.float32)
        return torch.mm(x, w.t())

    def linear_skinny(self, x: torch.Tensor, w: torch.Tensor, *, delta=None, norm_weight=None, eps: float = 0.0,
                      swiglu: bool = False, residual: Optional[torch.Tensor] = None):
        """The few-rows product (bf16, at most 16 rows) with its optional fused residual add, RMSNorm and
        SwiGLU in front and behind.  ``residual``: the result is ``round(round(x . w^T) + residual)``.  Returns
        ``out`` — or ``(x + delta, out)`` when ``delta`` is given — or None when the kernel does not take the shape."""
        M, K = x.shape
        N = w.shape[0]
        if (x.dtype != torch.bfloat16 or M > 16 or K % 32 or K > 16384 or x.stride(1) != 1 or w.stride(1) != 1
                or (swiglu and (N % 16 or residual is not None))
                or (residual is not None and (residual.shape != (M, N) or not residual.is_contiguous()))):
            return None
        out = torch.empty(M, N // 2 if swiglu else N, dtype=torch.bfloat16, device=x.device)
        x_out = torch.empty_like(x) if delta is not None else None
        nd = _DT[norm_weight.dtype] if norm_weight is not None else 0
        rc = self.lib.pih_gemm_skinny(_ptr(x), _ptr(delta), _ptr(x_out), nd, _ptr(norm_weight), c_float(eps), _ptr(w),
                                      _ptr(out), _ptr(residual), M, N, K, c_ll(x.stride(0)), c_ll(w.stride(0)),
                                      c_ll(out.stride(0)), 1 if swiglu else 0, self._err(), self._stream())
        if rc == -2:
            return None
        self._check(rc, "gemm_skinny")
        return out if delta is None else (x_out, out)

    def linear_add(self, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor):
        """``round(round(x . w^T) + residual)`` as one kernel — an output projection with the residual add that
        follows it — or None when only the separate kernels can do it (the caller then passes the product on and
        the next norm adds it)."""
        if x.shape[0] > self.skinny_max_rows or not self.fused_residual:
            return None
        return self.linear_skinny(x, w, residual=residual)

    def linear_tcgen05_swiglu(self, x: torch.Tensor, w: torch.Tensor):
        """``SwiGLU(x . w^T)`` with the pack's tcgen05 product on pairs of SMs and SiLU-mul in its epilogue: ``w``
        holds blocks of 8 gate rows followed by their 8 up rows; returns ``[M, N / 2]`` (bf16), or None for shapes
        that the kernel does not take."""
        M, K = x.shape
        N = w.shape[0]
        if x.dtype != torch.bfloat16 or N % 16 or x.stride(1) != 1 or w.stride(1) != 1:
            return None
        out = torch.empty(M, N // 2, dtype=torch.bfloat16, device=x.device)
        rc = self.lib.pih_gemm_tcgen05_pair(_DT[torch.bfloat16], _ptr(x), _ptr(w), _ptr(out), M, N, K,
                                            c_ll(x.stride(0)), c_ll(w.stride(0)), c_ll(out.stride(0)), 0, 1,
                                            self._err(), self._stream())
        if rc == -2:
            return None
        self._check(rc, "gemm_tcgen05_pair")
        return out

    def norm_linear(self, h: torch.Tensor, delta: Optional[torch.Tensor], norm_weight: torch.Tensor, eps: float,
                    w: torch.Tensor, swiglu_interleave: int = 0):
        """``h' = h + delta`` (when delta is given), ``out = rmsnorm(h') . w^T`` and, with
        ``swiglu_interleave``, SiLU-mul over gate/up column blocks of that size.  Returns ``(h', out)``;
        ``h'`` may be ``h`` updated in place or a new tensor.  One kernel for few rows, else the separate ones."""
        if h.dtype == torch.bfloat16 and h.shape[0] <= self.skinny_max_rows and swiglu_interleave in (0, 8):
            if delta is not None:
                res = self.linear_skinny(h, w, delta=delta, norm_weight=norm_weight, eps=eps,
                                         swiglu=swiglu_interleave == 8)
                if res is not None:
                    return res
            else:
                out = self.linear_skinny(h, w, norm_weight=norm_weight, eps=eps, swiglu=swiglu_interleave == 8)
                if out is not None:
                    return h, out
        xn = self.rmsnorm(h, norm_weight, eps, delta=delta)
        if (swiglu_interleave == 8 and xn.dtype == torch.bfloat16
                and self.lib.pih_pair_swiglu_wanted(xn.shape[0], w.shape[0])):
            out = self.linear_tcgen05_swiglu(xn, w)
            if out is not None:
                return h, out
        out = self.linear(xn, w)
        if swiglu_interleave:
            out = self.silu_mul(out, swiglu_interleave)
        return h, out

    def linear_tcgen05(self, x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                       tile_n: int = 0, pairs: bool = False):
        """The pack's tcgen05 / TMA product (bf16 in, fp32 accumulation).  Returns None when the
        operands cannot be described to TMA (K or a row stride not a multiple of 8).  ``pairs``: the kernel
        that puts two SMs on a 256-row tile (``tile_n`` 128 or 256)."""
        M, K = x.shape
        N = w.shape[0]
        out_dtype = out_dtype or x.dtype
        out = torch.empty(M, N, dtype=out_dtype, device=x.device)
        if pairs:
            rc = self.lib.pih_gemm_tcgen05_pair(_DT[out_dtype], _ptr(x), _ptr(w), _ptr(out), M, N, K,
                                                c_ll(x.stride(0)), c_ll(w.stride(0)), c_ll(N), tile_n, 0,
                                                self._err(), self._stream())
        else:
            rc = self.lib.pih_gemm_tcgen05(_DT[out_dtype], _ptr(x), _ptr(w), _ptr(out), M, N, K, c_ll(x.stride(0)),
                                           c_ll(w.stride(0)), c_ll(N), tile_n, self._err(), self._stream())
        if rc == -2:
            return None
        self._check(rc, "gemm_tcgen05")
        return out

    def linear_plain(self, x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """The pack's FMA product for any supported dtype (plain twin of the tensor-core products)."""
        M, K = x.shape
        N = w.shape[0]
        out_dtype = out_dtype or x.dtype
        out = torch.empty(M, N, dtype=out_dtype, device=x.device)
        rc = self.lib.pih_gemm_simt(_DT[x.dtype], _DT[out_dtype], _ptr(x), _ptr(w), _ptr(out), M, N, K,
                                    c_ll(x.stride(0)), c_ll(w.stride(0)), c_ll(N), self._stream())
        self._check(rc, "gemm_simt")
        return out

    def qk_norm_rope_kv_write(self, qkv, *, heads, kv_heads, head_dim, q_norm, k_norm, eps, rope_table,
                              rotary_dim, positions, slot_mapping, kv_cache, write_kv) -> None:
        """Per-head RMSNorm and rotation of the q and k heads of the rows ``[q | k | v]``; q is changed in place,
        and with ``write_kv`` k and v go to their slots of the cache.  The k part of the rows is not to be read
        afterwards: it holds the new k only where the kernel also wrote it there (few rows, rows without a slot)."""
        rows = qkv.shape[0]
        wd = _DT[q_norm.dtype] if q_norm is not None else _DT[qkv.dtype]
        num_pages, page_size = kv_cache.shape[0], kv_cache.shape[3]
        max_pos = rope_table.shape[0] if rope_table is not None else 0
        rc = self.lib.pih_qk_norm_rope_kv_write(
            _DT[qkv.dtype], wd, _ptr(qkv), qkv.stride(0), rows, heads, kv_heads, head_dim, _ptr(q_norm),
            _ptr(k_norm), c_float(eps), _ptr(rope_table), rotary_dim, max_pos, _ptr(positions),
            _ptr(slot_mapping), _ptr(kv_cache), page_size, num_pages, 1 if write_kv else 0, self._err(),
            self._stream())
        self._check(rc, "qk_norm_rope_kv_write")

    def paged_attention(self, qkv, *, heads, kv_heads, head_dim, kv_cache, block_table, step, scale,
                        window) -> torch.Tensor:
        """Attention of the step's rows over the cache.  bf16 runs on the tensor-core kernels
        when they have an instance for ``head_dim``; everything else on the generic kernel."""
        if self.tensor_core_attention and qkv.dtype == torch.bfloat16 and head_dim in self.MMA_HEAD_DIMS:
            return self.paged_attention_mma(qkv, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                            kv_cache=kv_cache, block_table=block_table, step=step,
                                            scale=scale, window=window)
        return self.paged_attention_generic(qkv, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                            kv_cache=kv_cache, block_table=block_table,
                                            request_of_row=step.request_of_row, positions=step.positions,
                                            scale=scale, window=window)

    MMA_HEAD_DIMS = (16, 32, 64, 80, 96, 128, 256)

    @staticmethod
    def attention_plan(host_cu_q, host_q_start, group: int):
        """(tile_max_q, dec_tok_cap, dec_max_ctx): a request is decode-like when it brings at most
        16 packed rows (rows * heads / kv_heads)."""
        tile_max_q = dec_cap = dec_ctx = 0
        for r in range(len(host_q_start)):
            n = host_cu_q[r + 1] - host_cu_q[r]
            if n * group <= 16:
                dec_cap = max(dec_cap, n)
                dec_ctx = max(dec_ctx, host_q_start[r] + n)
            else:
                tile_max_q = max(tile_max_q, n)
        return tile_max_q, dec_cap, dec_ctx

    def splits_for(self, num_requests: int, kv_heads: int, max_ctx: int = 0) -> int:
        """Splits per request of the decode attention: as many as fill the 2 x 148 CTA slots of the GPU in
        one wave (small batches are cut finely so that enough CTAs pull bandwidth, large ones not at all).
        Up to eight splits merge as a thread-block cluster, which is what a short context wants (the merge
        is most of its time); a long context wants every slot pulling (one request of 32768 keys: 69 us with
        8 splits, 34 us with 37), so beyond ``CLUSTER_MAX_KEYS`` keys per split the finer cut with the merge
        through scratch memory is taken.  A function of the batch size and the longest context that the
        step's block tables can hold, not of the contexts themselves: a captured step keeps its grid."""
        slots = (2 * 148) // max(1, num_requests * kv_heads)
        if self.cluster_attention and self.tma_attention and slots > 8 and max_ctx <= 8 * self.CLUSTER_MAX_KEYS:
            return 8                                   # one portable cluster per (request, kv head)
        return max(1, min(64, slots))

    CLUSTER_MAX_KEYS = 768

    def reserve_attention_scratch(self, num_requests, dec_tok_cap, heads, kv_heads, head_dim, max_ctx) -> None:
        """Make the split kernel's scratch large enough (before a CUDA graph that uses it is
        captured: an allocation cannot happen under capture).  A buffer that is outgrown is kept
        alive, because captured graphs hold its address."""
        splits = (-(-max_ctx // self.attention_split) if self.attention_split
                  else self.splits_for(num_requests, kv_heads, max_ctx))
        need = self.lib.pih_attention_scratch_floats(num_requests, dec_tok_cap, heads, kv_heads, head_dim, splits)
        if self._attn_scratch is None or self._attn_scratch.numel() < need:
            if self._attn_scratch is not None:
                self._retired_scratch.append(self._attn_scratch)     # captured graphs may still point at it
            # zeroed: the leading words are the kernel's tickets, which it leaves at zero
            self._attn_scratch = torch.zeros(int(need * 1.25) + 1024, dtype=torch.float32, device=self.device)

    def kv_tensor_map(self, kv_cache: torch.Tensor):
        """The TMA descriptor of one schedule entry's cache, made once; None when TMA cannot describe it."""
        key = (kv_cache.data_ptr(), tuple(kv_cache.shape))
        if key not in self._kv_maps:
            buf = ctypes.create_string_buffer(128)
            num_pages, _, kv_heads, page_size, head_dim = kv_cache.shape
            rc = self.lib.pih_make_kv_tensor_map(buf, _ptr(kv_cache), c_ll(num_pages), kv_heads, page_size, head_dim)
            self._kv_maps[key] = buf if rc == 0 else None
        return self._kv_maps[key]

    def paged_attention_mma(self, qkv, *, heads, kv_heads, head_dim, kv_cache, block_table, step, scale,
                            window, plan=None) -> torch.Tensor:
        rows = qkv.shape[0]
        group = heads // kv_heads
        plans = getattr(step, "attention_plans", None)
        if plan is None and plans is not None and group in plans:
            plan = plans[group]
        if plan is None:
            plan = self.attention_plan(step.host_cu_q, step.host_q_start, group)
            if plans is not None:
                plans[group] = plan
        tile_max_q, dec_cap, dec_ctx = plan
        out = torch.empty(rows, heads * head_dim, dtype=qkv.dtype, device=qkv.device)
        num_pages, page_size = kv_cache.shape[0], kv_cache.shape[3]
        split = self.attention_split                       # 0: cut on the device into `nsplits` parts
        nsplits = self.splits_for(step.num_requests, kv_heads, dec_ctx)
        max_ctx_ptr = getattr(step, "meta", None)
        if split == 0 and max_ctx_ptr is None:              # a caller without a packed batch: fix the cut here
            split = max(64, -(-(-(-max(dec_ctx, 1) // nsplits)) // 64) * 64)
        scratch = None
        if dec_cap > 0:
            self.reserve_attention_scratch(step.num_requests, dec_cap, heads, kv_heads, head_dim, dec_ctx)
            scratch = self._attn_scratch
        kv_map = self.kv_tensor_map(kv_cache) if (self.tma_attention or self.tcgen05_attention) else None
        if tile_max_q > 0 and self.tcgen05_attention and kv_map is not None and head_dim in (64, 128) \
                and page_size in (8, 16, 32, 64):
            rc = self.lib.pih_attention_prefill_tcgen05(
                _ptr(qkv), qkv.stride(0), rows, _ptr(out), _ptr(block_table), block_table.shape[1], _ptr(step.cu_q),
                _ptr(step.q_start), step.num_requests, tile_max_q, heads, kv_heads, head_dim, page_size, num_pages,
                c_float(scale), int(window), kv_map, self._err(), self._stream())
            self._check(rc, "attention_prefill_tcgen05")
            tile_max_q = 0                                  # done; what is left is decode-like
            if dec_cap == 0:
                return out
        rc = self.lib.pih_paged_attention_mma(
            _ptr(qkv), qkv.stride(0), _ptr(out), _ptr(kv_cache), _ptr(block_table), block_table.shape[1],
            _ptr(step.cu_q), _ptr(step.q_start), rows, step.num_requests, tile_max_q, dec_cap, dec_ctx, heads, kv_heads, head_dim, page_size, num_pages,
            c_float(scale), int(window), split, nsplits, _ptr(max_ctx_ptr), _ptr(scratch),
            kv_map if (self.tma_attention and dec_cap > 0) else None,
            self._err(), self._stream())
        self._check(rc, "paged_attention_mma")
        return out

    def qk_attention_fused(self, qkv, *, heads, kv_heads, head_dim, q_norm, k_norm, eps, rope_table, rotary_dim,
                           kv_cache, block_table, step, scale, window, write_kv):
        """``qk_norm_rope_kv_write`` and ``paged_attention`` as one kernel, for steps whose requests are all
        decode-like (bf16, the TMA split kernel's shapes, rotation over the whole head).  ``qkv`` stays raw.
        Returns the attention output, or None when the separate kernels have to run."""
        if (not self.fused_qk_attention or qkv.dtype != torch.bfloat16 or not self.tensor_core_attention
                or not self.tma_attention or (rope_table is not None and rotary_dim != head_dim)
                or (q_norm is not None and k_norm is not None and q_norm.dtype != k_norm.dtype)):
            return None
        group = heads // kv_heads
        plans = getattr(step, "attention_plans", None)
        plan = plans[group] if plans is not None and group in plans else None
        if plan is None:
            plan = self.attention_plan(step.host_cu_q, step.host_q_start, group)
            if plans is not None:
                plans[group] = plan
        tile_max_q, dec_cap, dec_ctx = plan
        max_ctx_ptr = getattr(step, "meta", None)
        if (tile_max_q > 0 or dec_cap <= 0 or (self.attention_split == 0 and max_ctx_ptr is None)
                or step.num_requests > self.fused_qk_max_requests):
            return None
        kv_map = self.kv_tensor_map(kv_cache)
        if kv_map is None:
            return None
        rows = qkv.shape[0]
        num_pages, page_size = kv_cache.shape[0], kv_cache.shape[3]
        nsplits = self.splits_for(step.num_requests, kv_heads, dec_ctx)
        self.reserve_attention_scratch(step.num_requests, dec_cap, heads, kv_heads, head_dim, dec_ctx)
        out = torch.empty(rows, heads * head_dim, dtype=qkv.dtype, device=qkv.device)
        norm = q_norm if q_norm is not None else k_norm
        rc = self.lib.pih_qk_attention_fused(
            _ptr(qkv), qkv.stride(0), _ptr(out), _ptr(kv_cache), _ptr(block_table), block_table.shape[1],
            _ptr(step.cu_q), _ptr(step.q_start), rows, step.num_requests, dec_cap, dec_ctx, heads, kv_heads, head_dim,
            page_size, num_pages, c_float(scale), int(window), self.attention_split, nsplits, _ptr(max_ctx_ptr),
            _ptr(self._attn_scratch), kv_map, _DT[norm.dtype] if norm is not None else 1, _ptr(q_norm), _ptr(k_norm),
            c_float(eps), _ptr(rope_table), rope_table.shape[0] if rope_table is not None else 0,
            1 if write_kv else 0, self._err(), self._stream())
        if rc == -2:
            return None
        self._check(rc, "qk_attention_fused")
        return out

    def paged_attention_generic(self, qkv, *, heads, kv_heads, head_dim, kv_cache, block_table,
                                request_of_row, positions, scale, window) -> torch.Tensor:
        rows = qkv.shape[0]
        out = torch.empty(rows, heads * head_dim, dtype=qkv.dtype, device=qkv.device)
        num_pages, page_size = kv_cache.shape[0], kv_cache.shape[3]
        rc = self.lib.pih_paged_attention_generic(
            _DT[qkv.dtype], _ptr(qkv), qkv.stride(0), _ptr(out), _ptr(kv_cache), _ptr(block_table),
            block_table.shape[1], _ptr(request_of_row), _ptr(positions), rows, heads, kv_heads, head_dim,
            page_size, num_pages, c_float(scale), int(window), self._err(), self._stream())
        self._check(rc, "paged_attention_generic")
        return out

    def silu_mul(self, gate_up: torch.Tensor, interleave: Optional[int] = None) -> torch.Tensor:
        """``silu(g) * u``; the columns of ``gate_up`` come in blocks of ``interleave`` gate columns
        followed by their up columns (default: all gates, then all ups)."""
        rows, two_i = gate_up.shape
        inter = two_i // 2
        out = torch.empty(rows, inter, dtype=gate_up.dtype, device=gate_up.device)
        rc = self.lib.pih_silu_mul(_DT[gate_up.dtype], _ptr(gate_up), _ptr(out), c_ll(rows), inter,
                                   interleave or inter, self._stream())
        self._check(rc, "silu_mul")
        return out

    def argmax(self, logits: torch.Tensor) -> torch.Tensor:
        rows, vocab = logits.shape
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
        scratch = torch.empty(rows * 128, dtype=torch.float32, device=logits.device) if vocab >= 8192 else None
        rc = self.lib.pih_argmax(_ptr(logits), rows, vocab, _ptr(out), _ptr(scratch), self._err(), self._stream())
        self._check(rc, "argmax")
        return out

    def selected_logprob(self, logits: torch.Tensor, tokens: torch.Tensor, fparams: Optional[torch.Tensor] = None,
                         iparams: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The log-probability of ``tokens[row]`` under each row's scaled logits (fp32 ``[rows]``); the
        parameters are those given to ``sample``, or none for greedy rows."""
        rows, vocab = logits.shape
        out = torch.empty(rows, dtype=torch.float32, device=logits.device)
        rc = self.lib.pih_selected_logprob(_ptr(logits), rows, vocab, _ptr(tokens), _ptr(fparams), _ptr(iparams),
                                           iparams.shape[1] if iparams is not None else 0, _ptr(out), self._err(),
                                           self._stream())
        self._check(rc, "selected_logprob")
        return out

    def top_logprobs(self, logits: torch.Tensor, count: int, fparams: Optional[torch.Tensor] = None,
                     iparams: Optional[torch.Tensor] = None):
        """The ``count`` (1 to 20) most probable ids of every row that are not suppressed — by value, then by id —
        and their log-probabilities under the row's scaled logits: ``(int32 [rows, count], fp32 [rows, count])``;
        the parameters are those given to ``sample``, or none for greedy rows."""
        rows, vocab = logits.shape
        words = self.lib.pih_top_logprobs_scratch_words(rows, vocab, count)
        if words < 0:
            raise ValueError(f"top_logprobs takes no vocabulary of {vocab}")
        scratch = torch.empty(max(int(words), 1), dtype=torch.float32, device=logits.device)
        ids = torch.empty(rows, count, dtype=torch.int32, device=logits.device)
        lps = torch.empty(rows, count, dtype=torch.float32, device=logits.device)
        rc = self.lib.pih_top_logprobs(_ptr(logits), rows, vocab, count, _ptr(fparams), _ptr(iparams),
                                       iparams.shape[1] if iparams is not None else 0, _ptr(ids), _ptr(lps),
                                       _ptr(scratch), self._err(), self._stream())
        self._check(rc, "top_logprobs")
        return ids, lps

    def sample(self, logits: torch.Tensor, fparams: torch.Tensor, iparams: torch.Tensor) -> torch.Tensor:
        rows, vocab = logits.shape
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
        rc = self.lib.pih_sample(_ptr(logits), rows, vocab, _ptr(fparams), _ptr(iparams), _ptr(out),
                                 self._err(), self._stream())
        self._check(rc, "sample")
        return out
