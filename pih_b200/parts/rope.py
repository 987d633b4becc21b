"""Rotary position encoding as a part: a table of (cos, sin) per position.

Angles as the reference's oracle computes them
(plugins/model-qwen3/qwen3_cpu_oracle.cpp:146-155): ``inv_i =
theta^(-2i/rotary_dim)``, ``angle = pos * inv_i`` in double, cast to
float32.  (Its GPU kernel uses float32 ``powf`` and has theta fixed in code,
kernels/cuda/qwen_bf16_primitives.cu:367-383; the two sides of the reference
differ there, and the double form is the one that does not drift at long
positions.)  The table is a pure function of the position, so cutting a
prompt into portions cannot change it.  The rotation itself (rotate-half
pairs ``(x_i, x_{i+rotary_dim/2})``, qwen_bf16_primitives.cu:326-347) is
done by the mixer's kernel, which reads this table.
"""
from __future__ import annotations

import torch

from .registry import Runtime, register_position

_TABLES = {}


@register_position("rope")
class RotaryEncoding:
    @classmethod
    def expected_tensors(cls, spec):
        return {}

    def __init__(self, spec, weights, rt: Runtime):
        if spec.rotary_dim % 2 or not 0 < spec.rotary_dim <= spec.head_dim:
            raise ValueError(f"rotary_dim must be even and within head_dim, got {spec.rotary_dim}")
        self.spec = spec
        self.rotary_dim = spec.rotary_dim
        key = (spec.rotary_dim, float(spec.theta), spec.max_positions, str(rt.device))
        if key not in _TABLES:
            pair = torch.arange(spec.rotary_dim // 2, dtype=torch.float64)
            inv = torch.pow(torch.tensor(float(spec.theta), dtype=torch.float64), -2.0 * pair / spec.rotary_dim)
            angle = torch.arange(spec.max_positions, dtype=torch.float64)[:, None] * inv[None, :]
            table = torch.stack([torch.cos(angle), torch.sin(angle)], dim=-1).to(torch.float32)
            _TABLES[key] = table.to(rt.device).contiguous()
        self._table = _TABLES[key]

    def rotation_table(self):
        """fp32 [max_positions, rotary_dim/2, 2] holding (cos, sin)."""
        return self._table
