"""Model parts: mixers, feed-forwards, norms, position encodings, blocks."""
from .registry import (PagedKVNeed, Runtime, StateNeed, TensorInfo, part_class, register_block,
                       register_ffn, register_mixer, register_norm, register_position, unregister)
from . import norm, rope, attention, swiglu, block  # noqa: F401  (registers the built-in kinds)

__all__ = ["PagedKVNeed", "Runtime", "StateNeed", "TensorInfo", "part_class", "register_block",
           "register_ffn", "register_mixer", "register_norm", "register_position", "unregister"]
