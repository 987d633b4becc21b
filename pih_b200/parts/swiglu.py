"""SwiGLU feed-forward: ``down( silu(gate(x)) * up(x) )``, no biases.

Reference order and rounding (plugins/model-qwen3/qwen3_bf16_execution_schedule.cpp:33-38;
kernels/cuda/qwen_bf16_primitives.cu:274-283): gate and up products are
rounded to the stream's dtype, ``(g / (1 + exp(-g))) * u`` is computed in
32-bit and rounded once, then the down product.  The reference runs gate and
up as two library products; here their weights are stacked (in blocks of 8
gate rows and their 8 up rows) so that one product reads the activations
once and can apply SiLU-mul in its epilogue.
"""
from __future__ import annotations

import torch

from .registry import Runtime, TensorInfo, register_ffn
from ._bind import bind_matrix


@register_ffn("swiglu")
class SwiGLU:
    pad_safe = True                        # row-wise: rows of padding are computed and never read

    @classmethod
    def expected_tensors(cls, spec):
        n = spec.names
        return {n["gate"]: TensorInfo((spec.intermediate, spec.hidden)),
                n["up"]: TensorInfo((spec.intermediate, spec.hidden)),
                n["down"]: TensorInfo((spec.hidden, spec.intermediate))}

    def __init__(self, spec, weights, rt: Runtime):
        if spec.activation != "silu":
            raise ValueError(f"SwiGLU supports activation 'silu', got {spec.activation!r}")
        self.spec = spec
        self.rt = rt
        n = spec.names
        gate, up = weights[n["gate"]], weights[n["up"]]
        # rows in blocks of 8 gate rows followed by their 8 up rows, so that a 16-row tile of the product
        # holds both halves of 8 outputs (the fused few-rows kernel applies SiLU-mul in its epilogue)
        self.interleave = 8 if spec.intermediate % 8 == 0 else spec.intermediate
        il = self.interleave
        stacked = torch.stack([gate.reshape(-1, il, spec.hidden), up.reshape(-1, il, spec.hidden)], dim=1)
        self.w_gate_up = bind_matrix(stacked.reshape(2 * spec.intermediate, spec.hidden), rt)
        self.w_down = bind_matrix(weights[n["down"]], rt)

    def forward(self, x):
        ops = self.rt.ops
        gate_up = ops.linear(x, self.w_gate_up)
        act = ops.silu_mul(gate_up, self.interleave)
        return ops.linear(act, self.w_down)

    def forward_prenorm(self, h, delta, norm):
        """``h' = h + delta; y = ffn(norm(h'))`` with the add, the norm and SiLU-mul fused into the
        gate-up product where the kernels can; returns ``(h', y)`` — or ``(h' + y, None)`` when the down product
        added the residual itself."""
        ops = self.rt.ops
        h, act = ops.norm_linear(h, delta, norm.weight, norm.spec.eps, self.w_gate_up,
                                 swiglu_interleave=self.interleave)
        if hasattr(ops, "linear_add"):
            h_new = ops.linear_add(act, self.w_down, h)      # the down product and the residual add as one kernel
            if h_new is not None:
                return h_new, None
        return h, ops.linear(act, self.w_down)
