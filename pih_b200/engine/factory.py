"""Puts a model folder, the kernels, a cache and the step function together."""
from __future__ import annotations

from typing import Optional

import torch

from ..cache import DEFAULT_PAGE_SIZE, CacheManager
from ..kernels import get_ops
from ..models import load_model
from ..parts.registry import Runtime
from .runner import ModelRunner

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def create_runner(model_dir: str, dtype: str = "bfloat16", *, device: str = "cuda:0", page_size: int = DEFAULT_PAGE_SIZE,
                  max_cache_tokens: int = 4096, max_requests: int = 32, cuda_graphs: bool = False,
                  ops: Optional[object] = None, capture_decode_after: int = 0):
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
                               max_requests=max_requests, cuda_graphs=cuda_graphs,
                               capture_decode_after=capture_decode_after)
    return config, model, cache, runner


def cache_tokens_for_memory(model, *, page_size: int, max_requests: int, max_batch_tokens: int, max_context: int,
                            memory_fraction: float = 0.9, free_and_total: Optional[tuple] = None) -> int:
    """How many tokens of cache fit on the model's device beside the weights that are already there.

    The reference fixes its pool at 2 560 pages of 16 tokens and takes the rest of its limits from a JSON file
    (plugins/model-qwen3/entrypoint.cpp:137-162, include/pih/model/qwen3_kv_slot_pool.h:52-58).  Here the
    pool is what the device has left: ``memory_fraction`` of its memory may be in use in all, of which the
    weights and whatever else is on the device now are part; from the remainder comes a workspace for a step
    of ``max_batch_tokens`` rows (activations of the widest block, logits for ``max_requests`` rows, the
    library's workspaces, CUDA graphs).  More than ``max_requests`` requests of ``max_context`` tokens is
    never needed.  Refuses when not even one request of ``max_context`` tokens fits."""
    if not 0.0 < memory_fraction <= 1.0:
        raise ValueError("memory_fraction must be in (0, 1]")
    rt, spec = model.rt, model.spec
    free, total = free_and_total if free_and_total is not None else torch.cuda.mem_get_info(rt.device)
    esize = torch.empty((), dtype=rt.dtype).element_size()
    per_token = 0
    widest = 4 * spec.hidden
    for entry, need in zip(spec.schedule, model.cache_needs()):
        if hasattr(need, "kv_heads"):
            per_token += 2 * need.kv_heads * need.head_dim * esize
    for block in spec.blocks:
        mixer, ffn = block.mixer, block.ffn
        widest = max(widest, 4 * spec.hidden + 2 * getattr(mixer, "q_size", 0) + 3 * getattr(mixer, "kv_size", 0)
                     + 3 * getattr(ffn, "intermediate", 0))
    workspace = max_batch_tokens * widest * esize + 6 * max_requests * spec.vocab * 4 + (768 << 20)
    budget = int(free - (1.0 - memory_fraction) * total - workspace)
    wanted = max_requests * (-(-max_context // page_size) * page_size)
    tokens = wanted if per_token == 0 else min(wanted, budget // per_token // page_size * page_size)
    if tokens < -(-max_context // page_size) * page_size:
        raise MemoryError(
            f"the device has {free / 2**30:.1f} GiB free of {total / 2**30:.1f}; with memory_fraction="
            f"{memory_fraction} and a workspace of {workspace / 2**30:.2f} GiB that leaves room for "
            f"{max(tokens, 0)} tokens of cache at {per_token} bytes a token, fewer than one request of "
            f"{max_context} tokens: lower maximum_context_tokens or maximum_batch_tokens, or give max_cache_tokens")
    return int(tokens)


def runner_for(model, *, page_size: int = DEFAULT_PAGE_SIZE, max_cache_tokens: int = 4096, max_requests: int = 32,
               cuda_graphs: bool = False, capture_decode_after: int = 0):
    """A cache and a step function for a model that is already built; returns ``(cache, runner)``."""
    rt = model.rt
    cache = CacheManager(model.cache_needs(), [e.reads_cache_of for e in model.spec.schedule],
                         page_size=page_size, num_pages=-(-max_cache_tokens // page_size),
                         max_requests=max_requests, device=rt.device, dtype=rt.dtype)
    return cache, ModelRunner(model, cache, cuda_graphs=cuda_graphs, capture_decode_after=capture_decode_after)
