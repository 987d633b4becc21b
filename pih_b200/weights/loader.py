"""Load a model folder's tensors by name and check them against what the model expects.

The reference validates every name, dtype and shape before it allocates
anything (src/model/resident_weight_set.cpp:32-57;
plugins/model-qwen3/artifact/qwen3_manifest.cpp:41-58) and reports the first
mismatch.  Here all problems are collected and raised as ONE
``WeightError`` that lists missing tensors, unexpected tensors and wrong
shapes, and nothing is returned unless the set is exactly right.

Tensors keep the dtype they are stored in: bfloat16 stays bfloat16, a tensor
stored in 32-bit stays 32-bit, integer tables become int32.  Conversion for
a compute path (for instance bf16 matrices widened for the 32-bit path) is
the parts' business when they bind their weights, never the loader's.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Mapping, Tuple

import torch

from .safetensors_io import SafetensorsFile

_FLOAT_OK = (torch.bfloat16, torch.float32)
_INT = (torch.int64, torch.int32, torch.int8, torch.uint8)


class WeightError(ValueError):
    """The model folder's tensors do not match the model."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_dtype=()):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)
        self.wrong_dtype = sorted(wrong_dtype)
        lines = ["weights do not match the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong dtype ({len(self.wrong_dtype)}): " + ", ".join(
                f"{n} is {got}" for n, got in self.wrong_dtype))
        super().__init__("\n".join(lines))


def _open_files(model_dir: str) -> Dict[str, SafetensorsFile]:
    """tensor name -> file that holds it; one file or an index of shards."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    files = {}
    if os.path.exists(single):
        f = SafetensorsFile(single)
        return {name: f for name in f.names()}
    if os.path.exists(index):
        with open(index, "r", encoding="utf-8") as fh:
            weight_map = json.load(fh)["weight_map"]
        opened = {}
        for name, shard in weight_map.items():
            if shard not in opened:
                opened[shard] = SafetensorsFile(os.path.join(model_dir, shard))
            if name in opened[shard].records:
                files[name] = opened[shard]
        # tensors present in a shard but not in the index are unexpected all the same
        for shard, f in opened.items():
            for name in f.names():
                files.setdefault(name, f)
        return files
    raise FileNotFoundError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json")


def load_weights(model_dir: str, expected: Mapping[str, Tuple[int, ...]],
                 optional: Mapping[str, Tuple[int, ...]] = ()) -> Dict[str, torch.Tensor]:
    """Return ``{name: cpu tensor}`` for exactly the ``expected`` names.

    ``optional`` names may be present or absent (a tied output head that a
    checkpoint stores anyway); when present their shape is checked too.
    """
    optional = dict(optional)
    files = _open_files(model_dir)
    try:
        missing = [n for n in expected if n not in files]
        unexpected = [n for n in files if n not in expected and n not in optional]
        wrong_shape, wrong_dtype = [], []
        for name, f in files.items():
            want = expected.get(name, optional.get(name))
            if want is None:
                continue
            rec = f.records[name]
            if tuple(rec.shape) != tuple(want):
                wrong_shape.append((name, tuple(rec.shape), tuple(want)))
            if rec.dtype not in _FLOAT_OK and rec.dtype not in _INT:
                wrong_dtype.append((name, str(rec.dtype)))
        if missing or unexpected or wrong_shape or wrong_dtype:
            raise WeightError(missing, unexpected, wrong_shape, wrong_dtype)
        out = {}
        for name in list(expected) + [n for n in optional if n in files]:
            t = files[name].read_tensor(name)
            if t.dtype in _INT:
                t = t.to(torch.int32)
            out[name] = t
        return out
    finally:
        for f in set(files.values()):
            f.close()
