"""Part specifications: what a model is made of, as plain data.

An architecture's typed configuration (``pih_b200.config.qwen3``) is turned
into a ``ModelSpec``: a list of ``BlockSpec`` (one per distinct layer, each
naming its mixer, feed-forward, norms and position encoding with every size
and constant as a field) and a ``schedule`` — the order in which layers run.
The parts in ``pih_b200.parts`` are built from these specs alone; none of
them knows which architecture it belongs to.

``kind`` strings are keys of the part registries in
``pih_b200.parts.registry``; a new kind of part brings its own spec class
(any dataclass with a ``kind`` field) and registers a builder for it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping, Optional, Sequence


def _names(**kw):
    return field(default_factory=lambda: dict(kw))


@dataclass(frozen=True)
class NormSpec:
    width: int
    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class RopeSpec:
    """Rotate-half rotary encoding over the first ``rotary_dim`` columns of a head."""
    head_dim: int
    rotary_dim: int
    theta: float
    max_positions: int
    kind: str = "rope"


@dataclass(frozen=True)
class AttentionSpec:
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    scale: float                      # applied to q.k after the dot product
    qk_norm_eps: Optional[float]      # None: no per-head q/k norm
    window: Optional[int]             # None: all keys; W: the last W keys
    position: Optional[RopeSpec]
    kind: str = "attention"
    # tensor names below the block's prefix, by role
    names: Mapping[str, str] = _names(q="self_attn.q_proj.weight", k="self_attn.k_proj.weight",
                                      v="self_attn.v_proj.weight", o="self_attn.o_proj.weight",
                                      q_norm="self_attn.q_norm.weight", k_norm="self_attn.k_norm.weight")

    @property
    def q_size(self) -> int:
        return self.heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.kv_heads * self.head_dim


@dataclass(frozen=True)
class SwiGLUSpec:
    hidden: int
    intermediate: int
    activation: str = "silu"
    kind: str = "swiglu"
    names: Mapping[str, str] = _names(gate="mlp.gate_proj.weight", up="mlp.up_proj.weight",
                                      down="mlp.down_proj.weight")


@dataclass(frozen=True)
class BlockSpec:
    """One layer: ``h += mixer(norm_in(h)); h += ffn(norm_post(h))`` for
    ``arrangement == "prenorm"``.  ``prefix`` is the layer's tensor-name
    prefix in the weight files."""
    prefix: str
    mixer: object
    ffn: object
    norm_in: NormSpec
    norm_post: NormSpec
    arrangement: str = "prenorm"
    names: Mapping[str, str] = _names(norm_in="input_layernorm.",
                                      norm_post="post_attention_layernorm.")


@dataclass(frozen=True)
class ScheduleEntry:
    """Run layer ``layer``.  ``reads_cache_of`` names an earlier entry of the
    schedule (by its index in the list) whose cache this entry's mixer reads
    instead of keeping one of its own."""
    layer: int
    reads_cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    vocab: int
    hidden: int
    blocks: Sequence[BlockSpec]
    schedule: Sequence[ScheduleEntry]
    final_norm: NormSpec
    tie_embeddings: bool
    embed_name: str = "model.embed_tokens.weight"
    final_norm_prefix: str = "model.norm."
    head_name: str = "lm_head.weight"
    max_positions: int = 0
    eos_token_ids: Sequence[int] = field(default_factory=tuple)

    def validate(self) -> None:
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.blocks):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, the model has {len(self.blocks)}")
            if e.reads_cache_of is not None:
                if not 0 <= e.reads_cache_of < i:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.reads_cache_of}, "
                                     "which must be an earlier entry")
                if self.schedule[e.reads_cache_of].reads_cache_of is not None:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.reads_cache_of}, "
                                     "which keeps none of its own")
