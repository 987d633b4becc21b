"""Typed configuration of the Qwen3 dense decoder, read from its config.json keys.

The reference's parser (plugins/model-qwen3/qwen3_config.cpp:53-135; struct
include/pih/model/qwen3_config.h:11-35) reads the same keys and then pins
every one of them to the 0.6B values.  This class keeps the keys and their
checks of meaning (no biases, no rope scaling, SiLU) and drops the pinning:
every size is a field, nothing is assumed in code.

One extension: the reference refuses ``use_sliding_window``
(qwen3_config.cpp:65-70); here, when it is true, layers with index
``>= max_window_layers`` attend to the last ``sliding_window`` keys only, so
that one model can hold layers with different cache needs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, asdict
from typing import Optional, Tuple

from .registry import register_architecture
from .specs import (AttentionSpec, BlockSpec, ModelSpec, NormSpec, RopeSpec,
                    ScheduleEntry, SwiGLUSpec)

_REQUIRED_INT = ("hidden_size", "intermediate_size", "num_hidden_layers",
                 "num_attention_heads", "num_key_value_heads", "vocab_size",
                 "max_position_embeddings")


def _as_int(raw: dict, key: str, minimum: int = 1) -> int:
    v = raw.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
        raise ValueError(f"config.json: {key!r} must be an integer >= {minimum}, got {v!r}")
    return v


def _as_number(raw: dict, key: str) -> float:
    v = raw.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or v <= 0:
        raise ValueError(f"config.json: {key!r} must be a positive number, got {v!r}")
    return float(v)


@register_architecture("Qwen3ForCausalLM")
@dataclass(frozen=True)
class Qwen3Config:
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rope_theta: float
    rms_norm_eps: float
    tie_word_embeddings: bool
    torch_dtype: str = "bfloat16"
    hidden_act: str = "silu"
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[object] = None     # an id, or a tuple of ids
    model_type: str = "qwen3"

    # -- reading ---------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen3Config":
        if raw.get("model_type", "qwen3") != "qwen3":
            raise ValueError(f"config.json: model_type must be 'qwen3', got {raw.get('model_type')!r}")
        for flag in ("attention_bias", "mlp_bias"):
            v = raw.get(flag)
            if v not in (None, False):
                raise ValueError(f"config.json: {flag} is not supported (projections have no bias)")
        if raw.get("rope_scaling") is not None:
            raise ValueError("config.json: rope_scaling is not supported (plain rotary encoding only)")
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ValueError(f"config.json: hidden_act must be 'silu', got {act!r}")
        dtype = raw.get("torch_dtype", raw.get("dtype", "bfloat16"))
        if dtype not in ("bfloat16", "float32"):
            raise ValueError(f"config.json: torch_dtype must be 'bfloat16' or 'float32', got {dtype!r}")
        ints = {k: _as_int(raw, k) for k in _REQUIRED_INT}
        heads = ints["num_attention_heads"]
        if "head_dim" in raw and raw["head_dim"] is not None:
            head_dim = _as_int(raw, "head_dim")
        else:
            if ints["hidden_size"] % heads:
                raise ValueError("config.json: head_dim is absent and hidden_size is not a multiple of "
                                 "num_attention_heads")
            head_dim = ints["hidden_size"] // heads
        tie = raw.get("tie_word_embeddings", False)
        if not isinstance(tie, bool):
            raise ValueError("config.json: tie_word_embeddings must be true or false")
        use_window = raw.get("use_sliding_window", False)
        if not isinstance(use_window, bool):
            raise ValueError("config.json: use_sliding_window must be true or false")
        window = max_window_layers = None
        if use_window:
            window = _as_int(raw, "sliding_window")
            max_window_layers = _as_int(raw, "max_window_layers", minimum=0)
        ids = {}
        for k in ("bos_token_id", "eos_token_id"):
            v = raw.get(k)
            if k == "eos_token_id" and isinstance(v, (list, tuple)) and v and \
                    all(isinstance(i, int) and not isinstance(i, bool) for i in v):
                v = tuple(v)                       # some checkpoints list several end-of-sequence ids
            elif v is not None and (isinstance(v, bool) or not isinstance(v, int)):
                raise ValueError(f"config.json: {k} must be an integer or null")
            ids[k] = v
        cfg = cls(head_dim=head_dim, rope_theta=_as_number(raw, "rope_theta"),
                  rms_norm_eps=_as_number(raw, "rms_norm_eps"), tie_word_embeddings=tie,
                  torch_dtype=dtype, hidden_act=act, use_sliding_window=use_window,
                  sliding_window=window, max_window_layers=max_window_layers, **ints, **ids)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError("num_attention_heads must be a multiple of num_key_value_heads "
                             f"({self.num_attention_heads} vs {self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ValueError(f"head_dim must be even for rotate-half RoPE, got {self.head_dim}")
        for k in ("bos_token_id", "eos_token_id"):
            v = getattr(self, k)
            for i in (v if isinstance(v, tuple) else () if v is None else (v,)):
                if not 0 <= i < self.vocab_size:
                    raise ValueError(f"{k}={i} is outside the vocabulary of {self.vocab_size}")

    def to_dict(self) -> dict:
        d = asdict(self)
        if isinstance(d["eos_token_id"], tuple):
            d["eos_token_id"] = list(d["eos_token_id"])
        d["architectures"] = [self.architecture]
        d["use_cache"] = True
        d["attention_bias"] = False
        d["rope_scaling"] = None
        if not self.use_sliding_window:
            d.pop("sliding_window"), d.pop("max_window_layers")
        return d

    # -- derived sizes (include/pih/model/qwen3_config.h:28-33) -----------
    @property
    def q_projection_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_projection_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def layer_window(self, layer: int) -> Optional[int]:
        if self.use_sliding_window and layer >= (self.max_window_layers or 0):
            return self.sliding_window
        return None

    # -- the model as parts -------------------------------------------------
    def model_spec(self) -> ModelSpec:
        """Pre-norm blocks of (GQA attention with per-head q/k RMSNorm and
        RoPE) and SwiGLU, final RMSNorm, output head tied or not
        (plugins/model-qwen3/qwen3_bf16_execution_schedule.cpp:19-64)."""
        # the reference computes the scale on the host in fp32:
        # plugins/model-qwen3/nvidia_qwen3_bf16_engine.cpp:371
        scale = 1.0 / math.sqrt(self.head_dim)
        rope = RopeSpec(head_dim=self.head_dim, rotary_dim=self.head_dim, theta=self.rope_theta,
                        max_positions=self.max_position_embeddings)
        norm = NormSpec(width=self.hidden_size, eps=self.rms_norm_eps)
        blocks = []
        for i in range(self.num_hidden_layers):
            attn = AttentionSpec(hidden=self.hidden_size, heads=self.num_attention_heads,
                                 kv_heads=self.num_key_value_heads, head_dim=self.head_dim,
                                 scale=scale, qk_norm_eps=self.rms_norm_eps,
                                 window=self.layer_window(i), position=rope)
            ffn = SwiGLUSpec(hidden=self.hidden_size, intermediate=self.intermediate_size,
                             activation=self.hidden_act)
            blocks.append(BlockSpec(prefix=f"model.layers.{i}.", mixer=attn, ffn=ffn,
                                    norm_in=norm, norm_post=norm))
        eos: Tuple[int, ...] = () if self.eos_token_id is None else (
            tuple(self.eos_token_id) if isinstance(self.eos_token_id, tuple) else (self.eos_token_id,))
        spec = ModelSpec(vocab=self.vocab_size, hidden=self.hidden_size, blocks=tuple(blocks),
                         schedule=tuple(ScheduleEntry(i) for i in range(self.num_hidden_layers)),
                         final_norm=norm, tie_embeddings=self.tie_word_embeddings,
                         max_positions=self.max_position_embeddings, eos_token_ids=eos)
        spec.validate()
        return spec
