"""RMSNorm as a part: ``y = (x / sqrt(mean(x^2) + eps)) * w``, rounded once.

Formula and rounding point: kernels/cuda/qwen_bf16_primitives.cu:285-324 of
the reference (oracle plugins/model-qwen3/qwen3_cpu_oracle.cpp:85-97): the
sum of squares, the reciprocal square root and both multiplications are in
32-bit; the weight multiplies directly.  ``add_forward`` fuses the residual
add that precedes a norm in a pre-norm block (reference: a separate kernel,
qwen_bf16_primitives.cu:264-272): the sum is formed in 32-bit, rounded to
the stream's dtype, stored back, and that rounded value is what is normed —
the same values as the two separate kernels give.
"""
from __future__ import annotations

from .registry import Runtime, TensorInfo, register_norm
from ._bind import bind_vector


@register_norm("rmsnorm")
class RMSNorm:
    fusable = True        # (weight, spec.eps) may be handed to an op that fuses this norm into a product

    @classmethod
    def expected_tensors(cls, spec):
        return {"weight": TensorInfo((spec.width,), "one_plus_normal")}

    def __init__(self, spec, weights, rt: Runtime):
        self.spec = spec
        self.rt = rt
        self.weight = bind_vector(weights["weight"], rt)

    def forward(self, x, rows=None):
        return self.rt.ops.rmsnorm(x, self.weight, self.spec.eps, delta=None, rows=rows)

    def add_forward(self, h, delta, rows=None):
        return self.rt.ops.rmsnorm(h, self.weight, self.spec.eps, delta=delta, rows=rows)
