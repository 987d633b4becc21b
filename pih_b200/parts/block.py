"""The arrangement of parts in a layer.

``prenorm``: ``h += mixer(norm_in(h)); h += ffn(norm_post(h))``
(plugins/model-qwen3/qwen3_bf16_execution_schedule.cpp:19-39).  The block
passes on the residual stream ``h`` together with ``delta``, the last
sub-layer's output that is not yet added, so that the add fuses with the
next norm wherever that norm lives (the next block's, or the model's final
norm).  ``delta`` is None when the last sub-layer has added its output itself
(for few rows the output projections add the residual in their epilogue).
"""
from __future__ import annotations

from .registry import Runtime, part_class, register_block


def _sub(weights, names, prefix=""):
    return {rel: weights[prefix + rel] for rel in names}


@register_block("prenorm")
class PreNormBlock:
    @classmethod
    def expected_tensors(cls, spec):
        out = {}
        n = spec.names
        for rel, info in part_class("norm", spec.norm_in.kind).expected_tensors(spec.norm_in).items():
            out[n["norm_in"] + rel] = info
        for rel, info in part_class("norm", spec.norm_post.kind).expected_tensors(spec.norm_post).items():
            out[n["norm_post"] + rel] = info
        out.update(part_class("mixer", spec.mixer.kind).expected_tensors(spec.mixer))
        out.update(part_class("ffn", spec.ffn.kind).expected_tensors(spec.ffn))
        return out

    def __init__(self, spec, weights, rt: Runtime):
        self.spec = spec
        self.rt = rt
        n = spec.names
        norm_in_cls = part_class("norm", spec.norm_in.kind)
        norm_post_cls = part_class("norm", spec.norm_post.kind)
        mixer_cls = part_class("mixer", spec.mixer.kind)
        ffn_cls = part_class("ffn", spec.ffn.kind)
        self.norm_in = norm_in_cls(
            spec.norm_in, _sub(weights, norm_in_cls.expected_tensors(spec.norm_in), n["norm_in"]), rt)
        self.norm_post = norm_post_cls(
            spec.norm_post, _sub(weights, norm_post_cls.expected_tensors(spec.norm_post), n["norm_post"]), rt)
        self.mixer = mixer_cls(spec.mixer, _sub(weights, mixer_cls.expected_tensors(spec.mixer)), rt)
        self.ffn = ffn_cls(spec.ffn, _sub(weights, ffn_cls.expected_tensors(spec.ffn)), rt)
        self._native_ok = None             # decided at the first step

    def forward(self, h, delta, step, cache):
        # kernels that can issue a whole block of these parts from one native call get it (the same kernels in the
        # same order as below; what they do not take comes back as None)
        if self._native_ok is None:
            native = getattr(self.rt.ops, "native_block", None)
            self._native_ok = native is not None and self.rt.ops._native_supports(self)
        if self._native_ok:
            done = self.rt.ops.native_block(self, h, delta, step, cache)
            if done is not None:
                return done
        # a part that can take "add, norm, then me" as one call gets it (fewer kernels for few rows);
        # any other part gets the normed rows
        fused_in = getattr(self.norm_in, "fusable", False)
        fused_post = getattr(self.norm_post, "fusable", False)
        if fused_in and hasattr(self.mixer, "forward_prenorm"):
            h, a = self.mixer.forward_prenorm(h, delta, self.norm_in, step, cache)
        else:
            a = self.mixer.forward(self.norm_in.add_forward(h, delta), step, cache)
        if fused_post and hasattr(self.ffn, "forward_prenorm"):
            return self.ffn.forward_prenorm(h, a, self.norm_post)
        return h, self.ffn.forward(self.norm_post.add_forward(h, a))
