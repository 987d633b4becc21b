"""Grouped-query causal attention over the paged cache, as a mixer.

Order of operations from the reference's schedule
(plugins/model-qwen3/qwen3_bf16_execution_schedule.cpp:19-39): q/k/v
products (rounded to the stream's dtype); per-head RMSNorm of q and k (rows
of ``head_dim``, one weight for all heads) before the rotation; rotate-half
RoPE on q and k; keys and values appended to the cache; attention over the
cache with the scale applied after the dot product and a 32-bit online
softmax (kernels/cuda/qwen_bf16_primitives.cu:660-733); the o product.
Query head ``h`` reads kv head ``h // (heads // kv_heads)``
(plugins/model-qwen3/qwen3_gqa_oracle.cpp:63; the reference's kernel has the
group size 2 fixed in code, qwen_bf16_primitives.cu:673).

The reference runs q, k and v as three library products and norm, rotation
and append as five kernels; here the three weights are stacked so that one
product reads the activations once, and one kernel norms, rotates and
writes the cache.  Every size and constant comes from the spec.
"""
from __future__ import annotations

import torch

from .registry import PagedKVNeed, Runtime, TensorInfo, part_class, register_mixer
from ._bind import bind_matrix, bind_vector


@register_mixer("attention")
class PagedAttention:
    # A step may be padded (rows of no request, requests without rows: see engine/batch.py); the kernels of this
    # part leave padding alone.  A mixer that does not say so is only given steps as they are.
    pad_safe = True

    @classmethod
    def expected_tensors(cls, spec):
        n = spec.names
        out = {n["q"]: TensorInfo((spec.q_size, spec.hidden)),
               n["k"]: TensorInfo((spec.kv_size, spec.hidden)),
               n["v"]: TensorInfo((spec.kv_size, spec.hidden)),
               n["o"]: TensorInfo((spec.hidden, spec.q_size))}
        if spec.qk_norm_eps is not None:
            out[n["q_norm"]] = TensorInfo((spec.head_dim,), "one_plus_normal")
            out[n["k_norm"]] = TensorInfo((spec.head_dim,), "one_plus_normal")
        return out

    def __init__(self, spec, weights, rt: Runtime):
        if spec.heads % spec.kv_heads:
            raise ValueError(f"heads ({spec.heads}) must be a multiple of kv_heads ({spec.kv_heads})")
        if spec.window is not None and spec.window < 1:
            raise ValueError(f"window must be >= 1, got {spec.window}")
        self.spec = spec
        self.rt = rt
        n = spec.names
        self.w_qkv = bind_matrix(torch.cat([weights[n["q"]], weights[n["k"]], weights[n["v"]]], dim=0), rt)
        self.w_o = bind_matrix(weights[n["o"]], rt)
        self.q_norm = self.k_norm = None
        if spec.qk_norm_eps is not None:
            self.q_norm = bind_vector(weights[n["q_norm"]], rt)
            self.k_norm = bind_vector(weights[n["k_norm"]], rt)
        self.position = None
        if spec.position is not None:
            self.position = part_class("position", spec.position.kind)(spec.position, {}, rt)

    def cache_need(self):
        return PagedKVNeed(self.spec.kv_heads, self.spec.head_dim, self.spec.window)

    def forward(self, x, step, cache):
        s, ops = self.spec, self.rt.ops
        if cache.writable:
            qkv = ops.linear(x, self.w_qkv)                 # [T, q_size + 2 kv_size]
        else:
            qkv = ops.linear(x, self.w_qkv[:s.q_size])      # another entry's cache: only q is needed
        return self._attend(qkv, step, cache)

    def forward_prenorm(self, h, delta, norm, step, cache):
        """``h' = h + delta; y = mixer(norm(h'))`` with the add and the norm fused into the q/k/v product
        where the kernels can; returns ``(h', y)``."""
        s, ops = self.spec, self.rt.ops
        w = self.w_qkv if cache.writable else self.w_qkv[:s.q_size]
        h, qkv = ops.norm_linear(h, delta, norm.weight, norm.spec.eps, w)
        return self._attend(qkv, step, cache, residual=h)

    def _attend(self, qkv, step, cache, residual=None):
        """Attention and the output projection.  With ``residual`` (the stream ``h``) returns ``(h', delta)``: either
        ``(h + projection, None)`` when one kernel did both, or ``(h, projection)`` for the next norm to add."""
        s, ops = self.spec, self.rt.ops
        table = self.position.rotation_table() if self.position is not None else None
        rotary = self.position.rotary_dim if self.position is not None else 0
        qk = dict(heads=s.heads, kv_heads=s.kv_heads, head_dim=s.head_dim, q_norm=self.q_norm, k_norm=self.k_norm,
                  eps=s.qk_norm_eps or 0.0, rope_table=table, rotary_dim=rotary)
        attn = None
        if hasattr(ops, "qk_attention_fused"):
            # a decode step: one kernel norms and rotates q and k, appends to the cache and attends
            attn = ops.qk_attention_fused(qkv, kv_cache=cache.kv, block_table=cache.block_table, step=step,
                                          scale=s.scale, window=s.window or 0, write_kv=cache.writable, **qk)
        if attn is None:
            ops.qk_norm_rope_kv_write(qkv, positions=step.positions, slot_mapping=cache.slot_mapping,
                                      kv_cache=cache.kv, write_kv=cache.writable, **qk)
            attn = ops.paged_attention(
                qkv, heads=s.heads, kv_heads=s.kv_heads, head_dim=s.head_dim,
                kv_cache=cache.kv, block_table=cache.block_table, step=step,
                scale=s.scale, window=s.window or 0)
        if residual is None:
            return ops.linear(attn, self.w_o)
        if hasattr(ops, "linear_add"):
            h_new = ops.linear_add(attn, self.w_o, residual)
            if h_new is not None:
                return h_new, None
        return residual, ops.linear(attn, self.w_o)
