"""Puts a model folder, the kernels, a cache and the step function together."""
from __future__ import annotations

from typing import Optional

import torch

from ..cache import CacheManager
from ..kernels import get_ops
from ..models import load_model
from ..parts.registry import Runtime
from .runner import ModelRunner

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def create_runner(model_dir: str, dtype: str = "bfloat16", *, device: str = "cuda:0", page_size: int = 16,
                  max_cache_tokens: int = 4096, max_requests: int = 32, cuda_graphs: bool = False,
                  ops: Optional[object] = None, pad_decode_to: int = 1):
    """Returns ``(config, model, cache, runner)``.

    ``max_cache_tokens`` sizes every cache group's pool: ``ceil(max_cache_tokens
    / page_size)`` pages.  ``ops`` is the kernel object (default: the CUDA
    kernel pack of ``device``).
    """
    if dtype not in DTYPES:
        raise ValueError(f"dtype must be one of {sorted(DTYPES)}, got {dtype!r}")
    dev = torch.device(device)
    rt = Runtime(device=dev, dtype=DTYPES[dtype], ops=ops if ops is not None else get_ops(dev))
    config, model = load_model(model_dir, rt)
    cache, runner = runner_for(model, page_size=page_size, max_cache_tokens=max_cache_tokens,
                               max_requests=max_requests, cuda_graphs=cuda_graphs, pad_decode_to=pad_decode_to)
    return config, model, cache, runner


def runner_for(model, *, page_size: int = 16, max_cache_tokens: int = 4096, max_requests: int = 32,
               cuda_graphs: bool = False, pad_decode_to: int = 1):
    """A cache and a step function for a model that is already built; returns ``(cache, runner)``."""
    rt = model.rt
    cache = CacheManager(model.cache_needs(), [e.reads_cache_of for e in model.spec.schedule],
                         page_size=page_size, num_pages=-(-max_cache_tokens // page_size),
                         max_requests=max_requests, device=rt.device, dtype=rt.dtype)
    return cache, ModelRunner(model, cache, cuda_graphs=cuda_graphs, pad_decode_to=pad_decode_to)
