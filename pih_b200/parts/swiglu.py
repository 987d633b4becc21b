"""SwiGLU feed-forward: ``down( silu(gate(x)) * up(x) )``, no biases.

Reference order and rounding (plugins/model-qwen3/qwen3_bf16_execution_schedule.cpp:33-38;
kernels/cuda/qwen_bf16_primitives.cu:274-283): gate and up products are
rounded to the stream's dtype, ``(g / (1 + exp(-g))) * u`` is computed in
32-bit and rounded once, then the down product.  The reference runs gate and
up as two library products; here their weights are stacked ``[gate; up]`` so
that one product reads the activations once.
"""
from __future__ import annotations

import torch

from .registry import Runtime, TensorInfo, register_ffn
from ._bind import bind_matrix


@register_ffn("swiglu")
class SwiGLU:
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
        self.w_gate_up = bind_matrix(torch.cat([weights[n["gate"]], weights[n["up"]]], dim=0), rt)
        self.w_down = bind_matrix(weights[n["down"]], rt)

    def forward(self, x):
        ops = self.rt.ops
        gate_up = ops.linear(x, self.w_gate_up)
        act = ops.silu_mul(gate_up)
        return ops.linear(act, self.w_down)
