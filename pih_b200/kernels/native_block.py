"""One native call per block: the argument records of ``csrc/block_native.cu`` and the code that fills them.

A pre-norm block of the built-in parts (RMSNorm, paged attention with rotary positions or none, SwiGLU) can be
run by ``pih_prenorm_attention_swiglu_block``: the same kernels in the same order as the parts issue them one
call at a time, from one call.  What is decided on the host — whether a step's requests are all decode-like,
how the decode attention is cut, which kernels take the head size — is decided here exactly as
``CudaOps.paged_attention_mma`` and ``CudaOps.qk_attention_fused`` decide it, once per step and attention
geometry, and handed over as plain numbers.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

c_void_p, c_int, c_float, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
_DT = {torch.float32: 0, torch.bfloat16: 1}


class StepArgs(ctypes.Structure):
    _fields_ = [("dtype", c_int), ("rows", c_int), ("num_requests", c_int), ("skinny_max_rows", c_int),
                ("fused_residual", c_int), ("positions", c_void_p), ("request_of_row", c_void_p), ("cu_q", c_void_p),
                ("q_start", c_void_p), ("max_ctx_ptr", c_void_p), ("error", c_void_p), ("stream", c_void_p),
                ("library_workspace", c_void_p), ("library_workspace_bytes", c_ll)]


class AttentionArgs(ctypes.Structure):
    _fields_ = [("block_table", c_void_p), ("slot_mapping", c_void_p), ("table_width", c_int), ("page_size", c_int),
                ("num_pages", c_int), ("tensor_cores", c_int), ("try_fused", c_int), ("tcgen05_prefill", c_int),
                ("tma_split", c_int), ("tile_max_q", c_int), ("dec_cap", c_int), ("dec_ctx", c_int), ("split", c_int),
                ("nsplits", c_int), ("scratch", c_void_p)]


class BlockArgs(ctypes.Structure):
    _fields_ = [("norm_in_w", c_void_p), ("norm_post_w", c_void_p), ("w_qkv", c_void_p), ("w_o", c_void_p),
                ("w_gate_up", c_void_p), ("w_down", c_void_p), ("q_norm_w", c_void_p), ("k_norm_w", c_void_p),
                ("rope", c_void_p), ("ld_qkv", c_ll), ("ld_o", c_ll), ("ld_gate_up", c_ll), ("ld_down", c_ll),
                ("norm_w_dtype", c_int), ("qk_norm_dtype", c_int), ("norm_in_eps", c_float), ("norm_post_eps", c_float),
                ("qk_eps", c_float), ("scale", c_float), ("hidden", c_int), ("heads", c_int), ("kv_heads", c_int),
                ("head_dim", c_int), ("intermediate", c_int), ("interleave", c_int), ("window", c_int),
                ("rotary_dim", c_int), ("max_pos", c_int), ("qkv_cols", c_int), ("kv_cache", c_void_p),
                ("kv_map", c_void_p), ("writable", c_int), ("h", c_void_p), ("delta", c_void_p), ("h_sum", c_void_p),
                ("h_sum2", c_void_p), ("xn", c_void_p), ("qkv", c_void_p), ("attn", c_void_p), ("o", c_void_p),
                ("h2", c_void_p), ("gate_up", c_void_p), ("act", c_void_p), ("y", c_void_p), ("h3", c_void_p),
                ("out_h", c_int), ("out_delta", c_int), ("launched", c_int)]


def _ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


class _StepState:
    """What the blocks of one step share: the step record, the workspaces (two sets of the tensors that leave a
    block, used in turn: a block's inputs are the outputs of the block before it) and the attention records."""

    def __init__(self):
        self.args = None
        self.sets = None
        self.shared = None
        self.turn = 0
        self.attention = {}


class NativeBlocks:
    LIBRARY_WORKSPACE_BYTES = 32 << 20

    def __init__(self, ops):
        self.ops = ops
        self.fn = ops.lib.pih_prenorm_attention_swiglu_block
        self.fn.restype = c_int
        self._library_workspace = None

    # -- what a block is made of, read once ---------------------------------------------------------------------
    @staticmethod
    def supports(block) -> bool:
        from ..parts.attention import PagedAttention
        from ..parts.norm import RMSNorm
        from ..parts.rope import RotaryEncoding
        from ..parts.swiglu import SwiGLU
        m = block.mixer
        return (type(block.norm_in) is RMSNorm and type(block.norm_post) is RMSNorm and type(m) is PagedAttention
                and type(block.ffn) is SwiGLU and (m.position is None or type(m.position) is RotaryEncoding)
                and block.norm_in.weight.dtype == block.norm_post.weight.dtype
                and (m.q_norm is None) == (m.k_norm is None)
                and (m.q_norm is None or m.q_norm.dtype == m.k_norm.dtype))

    def _static(self, block) -> BlockArgs:
        m, f = block.mixer, block.ffn
        s = m.spec
        a = BlockArgs()
        a.norm_in_w, a.norm_post_w = _ptr(block.norm_in.weight), _ptr(block.norm_post.weight)
        a.w_qkv, a.w_o, a.w_gate_up, a.w_down = _ptr(m.w_qkv), _ptr(m.w_o), _ptr(f.w_gate_up), _ptr(f.w_down)
        a.q_norm_w, a.k_norm_w = _ptr(m.q_norm), _ptr(m.k_norm)
        table = m.position.rotation_table() if m.position is not None else None
        a.rope = _ptr(table)
        a.ld_qkv, a.ld_o = m.w_qkv.stride(0), m.w_o.stride(0)
        a.ld_gate_up, a.ld_down = f.w_gate_up.stride(0), f.w_down.stride(0)
        a.norm_w_dtype = _DT[block.norm_in.weight.dtype]
        a.qk_norm_dtype = _DT[m.q_norm.dtype] if m.q_norm is not None else 1
        a.norm_in_eps, a.norm_post_eps = block.norm_in.spec.eps, block.norm_post.spec.eps
        a.qk_eps, a.scale = s.qk_norm_eps or 0.0, s.scale
        a.hidden, a.heads, a.kv_heads, a.head_dim = s.hidden, s.heads, s.kv_heads, s.head_dim
        a.intermediate, a.interleave = f.spec.intermediate, f.interleave
        a.window = s.window or 0
        a.rotary_dim = m.position.rotary_dim if m.position is not None else 0
        a.max_pos = table.shape[0] if table is not None else 0
        block._native_keep = table                       # (the record holds raw addresses)
        return a

    # -- what a step's blocks share ------------------------------------------------------------------------------
    def _step_state(self, step, h: torch.Tensor) -> _StepState:
        st = getattr(step, "_native", None)
        if st is None:
            st = _StepState()
            ops = self.ops
            if self._library_workspace is None:
                self._library_workspace = torch.empty(self.LIBRARY_WORKSPACE_BYTES, dtype=torch.uint8, device=h.device)
            a = StepArgs()
            a.dtype, a.rows, a.num_requests = _DT[h.dtype], h.shape[0], step.num_requests
            a.skinny_max_rows, a.fused_residual = ops.skinny_max_rows, 1 if ops.fused_residual else 0
            a.positions, a.request_of_row = _ptr(step.positions), _ptr(step.request_of_row)
            a.cu_q, a.q_start = _ptr(step.cu_q), _ptr(step.q_start)
            a.max_ctx_ptr = _ptr(getattr(step, "meta", None))
            a.error = ops.error_word.data_ptr()
            a.library_workspace = self._library_workspace.data_ptr()
            a.library_workspace_bytes = self.LIBRARY_WORKSPACE_BYTES
            st.args = a
            step._native = st
        return st

    def _workspaces(self, st: _StepState, block, h: torch.Tensor, qkv_cols: int):
        T, H = h.shape
        s, f = block.mixer.spec, block.ffn.spec
        key = (qkv_cols, s.q_size, f.intermediate)
        if st.shared is None or st.shared["key"] != key:
            new = lambda cols: torch.empty(T, cols, dtype=h.dtype, device=h.device)
            st.shared = {"key": key, "xn": new(H), "qkv": new(qkv_cols), "attn": new(s.q_size),
                         "gate_up": new(2 * f.intermediate), "act": new(f.intermediate)}
            st.sets = [{n: new(H) for n in ("h_sum", "h_sum2", "o", "h2", "y", "h3")} for _ in range(2)]
        st.turn ^= 1
        return st.shared, st.sets[st.turn]

    def _attention(self, st: _StepState, step, spec, cache, h: torch.Tensor) -> AttentionArgs:
        ops = self.ops
        key = (cache.block_table.data_ptr(), spec.heads, spec.kv_heads, spec.head_dim)
        a = st.attention.get(key)
        if a is not None:
            return a
        a = AttentionArgs()
        num_pages, page_size = cache.kv.shape[0], cache.kv.shape[3]
        a.block_table, a.slot_mapping = _ptr(cache.block_table), _ptr(cache.slot_mapping)
        a.table_width, a.page_size, a.num_pages = cache.block_table.shape[1], page_size, num_pages
        bf16 = h.dtype == torch.bfloat16
        a.tensor_cores = 1 if (ops.tensor_core_attention and bf16 and spec.head_dim in ops.MMA_HEAD_DIMS) else 0
        if a.tensor_cores:
            group = spec.heads // spec.kv_heads
            plans = getattr(step, "attention_plans", None)
            plan = plans[group] if plans is not None and group in plans else None
            if plan is None:
                plan = ops.attention_plan(step.host_cu_q, step.host_q_start, group)
                if plans is not None:
                    plans[group] = plan
            tile_max_q, dec_cap, dec_ctx = plan
            a.tile_max_q, a.dec_cap, a.dec_ctx = tile_max_q, dec_cap, dec_ctx
            meta = getattr(step, "meta", None)
            split = ops.attention_split
            nsplits = ops.splits_for(step.num_requests, spec.kv_heads, dec_ctx)
            if split == 0 and meta is None:
                split = max(64, -(-(-(-max(dec_ctx, 1) // nsplits)) // 64) * 64)
            a.split, a.nsplits = split, nsplits
            if dec_cap > 0:
                ops.reserve_attention_scratch(step.num_requests, dec_cap, spec.heads, spec.kv_heads, spec.head_dim, dec_ctx)
                a.scratch = ops._attn_scratch.data_ptr()
            a.tcgen05_prefill = 1 if (tile_max_q > 0 and ops.tcgen05_attention and spec.head_dim in (64, 128)
                                      and page_size in (8, 16, 32, 64)) else 0
            a.tma_split = 1 if ops.tma_attention else 0
            a.try_fused = 1 if (ops.fused_qk_attention and ops.tma_attention and tile_max_q == 0 and dec_cap > 0
                                and not (ops.attention_split == 0 and meta is None)
                                and step.num_requests <= ops.fused_qk_max_requests) else 0
        st.attention[key] = a
        return a

    # -- one block -----------------------------------------------------------------------------------------------
    def run(self, block, h: torch.Tensor, delta: Optional[torch.Tensor], step, cache):
        """``(h', delta')`` of the block, or None when this path does not take it (the parts then run it)."""
        if not h.is_contiguous() or (delta is not None and not delta.is_contiguous()) or h.dtype not in _DT:
            return None
        # Steps of many rows in bfloat16 whose row count is their own stay with the parts: their products are the
        # library's, and called through torch a product of a row count not seen before costs far less host time
        # than through cublasGemmEx (which searches and loads anew for every new shape: measured on a serving run
        # whose portions all differ in length, 3.7 against 4.7 thousand generated tokens a second).  Few rows —
        # decode steps, where the host time of an uncaptured step matters most —, the 32-bit path (no library
        # product) and steps padded to a shape that comes again are issued from here.
        if (h.dtype == torch.bfloat16 and h.shape[0] > self.ops.skinny_max_rows
                and not getattr(step, "padded", False)):
            return None
        b = getattr(block, "_native_args", None)
        if b is None:
            b = block._native_args = self._static(block)
        ops = self.ops
        st = self._step_state(step, h)
        st.args.stream = torch._C._cuda_getCurrentRawStream(ops._device_index)
        spec = block.mixer.spec
        b.writable = 1 if cache.writable else 0
        b.qkv_cols = spec.q_size + (2 * spec.kv_size if cache.writable else 0)
        shared, mine = self._workspaces(st, block, h, b.qkv_cols)
        att = self._attention(st, step, spec, cache, h)
        b.kv_cache = cache.kv.data_ptr()
        kv_map = ops.kv_tensor_map(cache.kv) if (att.tensor_cores and (ops.tma_attention or ops.tcgen05_attention)) else None
        b.kv_map = ctypes.addressof(kv_map) if kv_map is not None else 0
        b.h, b.delta = h.data_ptr(), _ptr(delta)
        b.h_sum, b.h_sum2, b.o, b.h2 = (mine[n].data_ptr() for n in ("h_sum", "h_sum2", "o", "h2"))
        b.y, b.h3 = mine["y"].data_ptr(), mine["h3"].data_ptr()
        b.xn, b.qkv, b.attn = shared["xn"].data_ptr(), shared["qkv"].data_ptr(), shared["attn"].data_ptr()
        b.gate_up, b.act = shared["gate_up"].data_ptr(), shared["act"].data_ptr()
        rc = self.fn(ctypes.byref(st.args), ctypes.byref(att), ctypes.byref(b))
        if rc != 0:
            from .ops import KernelError
            raise KernelError(f"native block: a kernel was refused or failed ({rc})")
        ops.launches += b.launched
        h_out = (h, mine["h_sum"], mine["h2"], mine["h3"], mine["h_sum2"])[b.out_h]
        d_out = (None, mine["o"], mine["y"])[b.out_delta]
        return h_out, d_out
