"""The step function's host side on the CPU: real config, loader, parts, cache
manager and batch builder, with a torch stand-in for the kernels
(tests/fake_ops.py).  Every way of cutting the same requests into steps must
give the plain implementation's logits; a difference here is a fault of the
block tables, slot mappings or request bookkeeping, not of a kernel."""
import pytest
import torch

import plain_impl
import traces
from conftest import load_plain_weights
from fake_ops import FakeOps
from pih_b200.engine.factory import create_runner

LENGTHS = {"A": [70, 45, 90, 33, 61, 50, 77, 40], "B": [64, 33, 97, 41, 80, 55, 35, 66]}
PAGE = {"A": 16, "B": 8}


def _reference(model_dir, requests):
    cfg, w = load_plain_weights(model_dir)
    return {rid: plain_impl.forward(cfg, w, toks) for rid, toks in requests.items()}


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("family", ["whole", "tail_decode", "portions", "mixed"])
def test_cut_invariance_with_stand_in_kernels(model_dirs, tiny_configs, name, family):
    requests = traces.make_requests(tiny_configs[name]["vocab_size"], LENGTHS[name], seed=11)
    steps = getattr(traces, family)(requests)
    pool = traces.peak_tokens(steps, round_to=64)
    _, _, cache, runner = create_runner(model_dirs[name], "float32", device="cpu", page_size=PAGE[name],
                                        max_cache_tokens=pool, max_requests=4, ops=FakeOps())
    got = traces.replay(runner, steps)
    ref = _reference(model_dirs[name], requests)
    for rid in requests:
        err = float((got[rid].double() - ref[rid]).abs().max())
        assert err < 2e-5, f"{family} {rid}: max abs error {err}"
    cache.check()
    assert all(f == cache.num_pages for f in cache.num_free_pages()), "pages were lost"
    if family == "mixed":
        # the pool is smaller than what all requests need together: pages were used again
        assert all(g.pool.pages_handed_out > g.pool.num_pages for g in cache.groups)


def test_schedule_may_repeat_a_layer_and_share_a_cache(model_dirs, tiny_configs):
    """The order of layers is data: run layer 0 twice, and let the last entry read entry 0's cache."""
    from dataclasses import replace
    from pih_b200.cache import CacheManager
    from pih_b200.config import ScheduleEntry, config_from_dict
    from pih_b200.engine import ModelRunner, StepEntry
    from pih_b200.models import CausalLM
    from pih_b200.parts import Runtime

    cfg_raw, w64 = load_plain_weights(model_dirs["A"])
    config = config_from_dict(tiny_configs["A"])
    schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, reads_cache_of=0))
    spec = replace(config.model_spec(), schedule=schedule)
    rt = Runtime(torch.device("cpu"), torch.float32, FakeOps())
    model = CausalLM(spec, {k: v.float() for k, v in w64.items()}, rt)
    cache = CacheManager(model.cache_needs(), [e.reads_cache_of for e in schedule], page_size=16,
                         num_pages=8, max_requests=2, device=rt.device, dtype=rt.dtype)
    runner = ModelRunner(model, cache)
    toks = traces.make_requests(256, [50], seed=5)["r0"]
    ref = plain_impl.forward(cfg_raw, w64, toks, schedule=[(0, None), (1, None), (0, None), (1, 0)])
    rows = [runner.step([StepEntry("x", toks[:31], list(range(31)))]),
            runner.step([StepEntry("x", toks[31:], list(range(19)))])]
    err = float((torch.cat(rows).double() - ref).abs().max())
    assert err < 2e-5, err
    assert len(cache.groups) == 1 and len(cache.groups[0].entries) == 3
