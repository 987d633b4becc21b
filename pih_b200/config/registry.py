"""One registry from an architecture's name to its configuration class.

The reference selects its model plugin through a lock file and then insists
that ``architectures == ["Qwen3ForCausalLM"]``
(plugins/model-qwen3/qwen3_config.cpp:84-90; plugin lookup in
src/microkernel/plugin_registry.cpp:30-54).  Here the name in config.json is
the key: ``architectures[0]`` maps to a configuration class whose
``from_dict`` reads the architecture's own keys and whose ``model_spec``
describes the model as parts.
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict

_ARCHITECTURES: Dict[str, type] = {}


def register_architecture(name: str) -> Callable[[type], type]:
    def deco(cls: type) -> type:
        if name in _ARCHITECTURES and _ARCHITECTURES[name] is not cls:
            raise ValueError(f"architecture {name!r} is already registered")
        _ARCHITECTURES[name] = cls
        cls.architecture = name
        return cls
    return deco


def registered_architectures():
    return sorted(_ARCHITECTURES)


def config_class_for(name: str) -> type:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ValueError(f"unknown architecture {name!r}; registered: {registered_architectures()}") from None


def config_from_dict(raw: dict):
    archs = raw.get("architectures")
    if not isinstance(archs, list) or len(archs) != 1 or not isinstance(archs[0], str):
        raise ValueError("config.json: 'architectures' must be a list with exactly one name")
    return config_class_for(archs[0]).from_dict(raw)


def load_config(model_dir: str):
    path = os.path.join(model_dir, "config.json")
    with open(path, "r", encoding="utf-8") as f:
        raw = json.load(f)
    if not isinstance(raw, dict):
        raise ValueError(f"{path}: must hold a JSON object")
    return config_from_dict(raw)
