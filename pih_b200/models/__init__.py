"""A causal language model put together from parts, driven by a ``ModelSpec``.

``CausalLM`` owns the embedding table, the blocks, the final norm and the
output head; the order in which layers run is ``spec.schedule`` (a list that
may name a layer twice, or let an entry read an earlier entry's cache).
Order of the whole pass from the reference's schedule
(plugins/model-qwen3/qwen3_bf16_execution_schedule.cpp:51-63): embedding,
the layers, final norm, gather of the rows whose logits are wanted, output
head with 32-bit logits (src/backend/cuda/gemm_plan.cpp:111-113).  The
reference norms every row and gathers afterwards
(kernels/cuda/qwen_bf16_primitives.cu:736-759); here only the wanted rows
are normed, which gives the same values for those rows.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.registry import load_config
from ..config.specs import ModelSpec
from ..parts import part_class
from ..parts.registry import Runtime, TensorInfo
from ..parts._bind import bind_matrix
from ..weights.loader import load_weights


def expected_tensors(spec: ModelSpec) -> Dict[str, TensorInfo]:
    """Every tensor the model reads, by its name in the weight files."""
    out = {spec.embed_name: TensorInfo((spec.vocab, spec.hidden))}
    for block in spec.blocks:
        cls = part_class("block", block.arrangement)
        for rel, info in cls.expected_tensors(block).items():
            out[block.prefix + rel] = info
    norm_cls = part_class("norm", spec.final_norm.kind)
    for rel, info in norm_cls.expected_tensors(spec.final_norm).items():
        out[spec.final_norm_prefix + rel] = info
    if not spec.tie_embeddings:
        out[spec.head_name] = TensorInfo((spec.vocab, spec.hidden))
    return out


class CausalLM:
    def __init__(self, spec: ModelSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        spec.validate()
        self.spec = spec
        self.rt = rt
        self.embed = bind_matrix(weights[spec.embed_name], rt)
        self.head = self.embed if spec.tie_embeddings else bind_matrix(weights[spec.head_name], rt)
        self.blocks = []
        for block in spec.blocks:
            cls = part_class("block", block.arrangement)
            rel = {name: weights[block.prefix + name] for name in cls.expected_tensors(block)}
            self.blocks.append(cls(block, rel, rt))
        norm_cls = part_class("norm", spec.final_norm.kind)
        self.final_norm = norm_cls(
            spec.final_norm,
            {name: weights[spec.final_norm_prefix + name] for name in norm_cls.expected_tensors(spec.final_norm)},
            rt)

    @property
    def pad_safe(self) -> bool:
        """Whether a step may be padded to a larger shape: every mixer and feed-forward has to leave padding alone."""
        return all(getattr(b.mixer, "pad_safe", False) and getattr(b.ffn, "pad_safe", False) for b in self.blocks)

    # -- what the cache manager must provide, per schedule entry -------------
    def cache_needs(self) -> List[Optional[object]]:
        needs = []
        for entry in self.spec.schedule:
            if entry.reads_cache_of is not None:
                needs.append(None)
            else:
                needs.append(self.blocks[entry.layer].mixer.cache_need())
        return needs

    # -- one pass over the rows of a step --------------------------------------
    def forward(self, step, caches) -> Optional[torch.Tensor]:
        """``step``: the packed batch; ``caches[i]``: the cache view of
        schedule entry i.  Returns fp32 logits ``[len(step.logit_rows), vocab]``
        or None when no logits are wanted."""
        ops = self.rt.ops
        h = ops.embedding(self.embed, step.token_ids)
        delta = None
        for i, entry in enumerate(self.spec.schedule):
            h, delta = self.blocks[entry.layer].forward(h, delta, step, caches[i])
        if step.num_logit_rows == 0:
            return None
        xn = self.final_norm.add_forward(h, delta, rows=step.logit_rows)
        return ops.linear(xn, self.head, out_dtype=torch.float32)


def load_model(model_dir: str, rt: Runtime):
    """config.json -> registered configuration -> spec -> weights -> CausalLM."""
    config = load_config(model_dir)
    spec = config.model_spec()
    expected = {n: i.shape for n, i in expected_tensors(spec).items()}
    optional = {spec.head_name: (spec.vocab, spec.hidden)} if spec.tie_embeddings else {}
    weights = load_weights(model_dir, expected, optional)
    return config, CausalLM(spec, weights, rt)
