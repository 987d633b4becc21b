"""Registries of part kinds, and the interface each kind of part has.

A part is built from its spec alone (``spec.kind`` selects the class), gets
its weights by role, and is run by the block that holds it.  No part knows
which model it is in.

Interfaces
----------
Every part class has::

    expected_tensors(spec) -> {relative name: TensorInfo}    (classmethod)
    __init__(spec, weights: {relative name: tensor}, rt: Runtime)

and then, by family:

norm          ``forward(x) -> y`` and ``add_forward(h, delta) -> y`` which
              first does ``h += delta`` in place (delta may be None) and may
              restrict itself to ``rows`` (an int32 index tensor).
position      ``rotation_table() -> fp32 [max_positions, rotary_dim/2, 2]``
              (cos, sin) or None, and ``rotary_dim``; used by a mixer that
              rotates q and k.  Must be a pure function of the position.
mixer         ``cache_need() -> PagedKVNeed | StateNeed | None`` and
              ``forward(x, step, cache) -> y`` with x, y ``[T, hidden]``;
              ``step`` is the engine's ``StepBatch`` (packed rows, request
              boundaries ``cu_q``, positions, state slots), ``cache`` the
              view that the cache manager made for this schedule entry.
feed-forward  ``forward(x) -> y`` with x, y ``[T, hidden]``.
block         ``forward(h, delta, step, cache) -> (h, delta)``: the residual
              stream and the last sub-layer's output that is not added yet.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional, Tuple

import torch


@dataclass(frozen=True)
class TensorInfo:
    shape: Tuple[int, ...]
    init: str = "normal"          # "normal" | "one_plus_normal" (random-weights mode)


@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values per token.  ``window`` None: all keys are kept."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size, kept in a state slot."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class Runtime:
    """What a part needs to run: the device, the compute dtype and the kernels."""
    device: torch.device
    dtype: torch.dtype            # torch.bfloat16 (serving) or torch.float32 (true 32-bit path)
    ops: object


_REGISTRIES: Dict[str, Dict[str, type]] = {k: {} for k in ("norm", "position", "mixer", "ffn", "block")}


def _register(family: str, kind: str) -> Callable[[type], type]:
    def deco(cls: type) -> type:
        reg = _REGISTRIES[family]
        if kind in reg and reg[kind] is not cls:
            raise ValueError(f"{family} kind {kind!r} is already registered")
        reg[kind] = cls
        return cls
    return deco


def register_norm(kind: str):
    return _register("norm", kind)


def register_position(kind: str):
    return _register("position", kind)


def register_mixer(kind: str):
    return _register("mixer", kind)


def register_ffn(kind: str):
    return _register("ffn", kind)


def register_block(kind: str):
    return _register("block", kind)


def part_class(family: str, kind: str) -> type:
    try:
        return _REGISTRIES[family][kind]
    except KeyError:
        raise ValueError(f"unknown {family} kind {kind!r}; registered: {sorted(_REGISTRIES[family])}") from None


def unregister(family: str, kind: str) -> None:
    _REGISTRIES[family].pop(kind, None)
