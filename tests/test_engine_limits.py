"""The default size of the cache pool comes from the device's memory, not from a constant."""
import pytest
import torch

from fake_ops import FakeOps
from pih_b200.engine.factory import cache_tokens_for_memory
from pih_b200.models import load_model
from pih_b200.parts import Runtime

GiB = 1 << 30


def _model(model_dirs, name):
    rt = Runtime(torch.device("cpu"), torch.bfloat16, FakeOps())
    return load_model(model_dirs[name], rt)[1]


def test_pool_is_what_memory_leaves_and_never_more_than_the_requests_need(model_dirs, tiny_configs):
    model = _model(model_dirs, "B")
    cfg = tiny_configs["B"]
    per_token = cfg["num_hidden_layers"] * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2
    kw = dict(page_size=16, max_requests=32, max_batch_tokens=4096, max_context=1024)
    # plenty of memory: the cap is what 32 requests of 1024 tokens need
    assert cache_tokens_for_memory(model, free_and_total=(170 * GiB, 180 * GiB), **kw) == 32 * 1024
    # little memory: 10 % of the device stays free, a workspace comes off, the rest is pages
    kw["max_requests"] = 2048                               # (a tiny model: it takes many requests to fill 2 GiB)
    small = (3 * GiB // 2, 2 * GiB)
    tokens = cache_tokens_for_memory(model, free_and_total=small, **kw)
    assert 1024 <= tokens < 2048 * 1024 and tokens % 16 == 0
    assert tokens * per_token <= small[0] - small[1] // 10 - (768 << 20)
    # a larger fraction gives more pages, a larger step workspace fewer
    more = cache_tokens_for_memory(model, free_and_total=small, memory_fraction=0.95, **kw)
    fewer = cache_tokens_for_memory(model, free_and_total=small, **dict(kw, max_batch_tokens=65536))
    assert fewer < tokens < more


def test_pool_refuses_when_not_one_request_fits(model_dirs):
    model = _model(model_dirs, "A")
    with pytest.raises(MemoryError, match="fewer than one request of 512 tokens"):
        cache_tokens_for_memory(model, page_size=16, max_requests=4, max_batch_tokens=64, max_context=512,
                                free_and_total=(1 * GiB, 80 * GiB))
    with pytest.raises(ValueError):
        cache_tokens_for_memory(model, page_size=16, max_requests=4, max_batch_tokens=64, max_context=512,
                                memory_fraction=0.0, free_and_total=(1 * GiB, 80 * GiB))
