"""The scheduler's decisions, with a scripted step function instead of a model (as the
reference tests its controller with fake backends: tests/cpp/scheduler/controller_runtime_test.cpp)."""
import torch

from pih_b200.cache import CacheManager
from pih_b200.engine import Request, Scheduler
from pih_b200.parts import PagedKVNeed
from pih_b200.sampling import SamplingParams

import pytest


def make(num_pages=64, page_size=4, seqs=4, budget=16, max_context=None):
    cache = CacheManager([PagedKVNeed(1, 4, None)], [None], page_size=page_size, num_pages=num_pages,
                         max_requests=seqs, device=torch.device("cpu"), dtype=torch.float32,
                         allocate_tensors=False)
    return cache, Scheduler(cache, max_batch_sequences=seqs, max_batch_tokens=budget, max_context=max_context)


def run_step(cache, sched, token_of=lambda req: 100 + len(req.outputs)):
    """What the engine does around the model: append, commit, sample (scripted), update."""
    out = sched.schedule()
    for s in out.scheduled:
        cache.append(s.request.rid, len(s.tokens))
        cache.commit(s.request.rid)
    sampled = [token_of(s.request) if s.samples else None for s in out.scheduled]
    finished = sched.update(out, sampled)
    cache.check()
    return out, finished


def req(rid, n_prompt, **kw):
    return Request(rid, list(range(1, n_prompt + 1)), SamplingParams(**kw), eos_token_ids=(2,))


def test_prompt_is_cut_under_the_token_budget_and_decode_follows():
    cache, sched = make(budget=16)
    r = req("a", 40, max_tokens=3)
    sched.add(r)
    sizes = []
    while sched.has_work():
        out, _ = run_step(cache, sched)
        sizes.append([(len(s.tokens), s.samples) for s in out.scheduled])
    assert sizes == [[(16, False)], [(16, False)], [(8, True)], [(1, True)], [(1, True)]]
    assert r.outputs == [100, 101, 102] and r.finish_reason == "length"
    # ledger of the reference: K = P + A - 1 after every decode step
    assert r.num_computed == 40 + 3 - 1
    assert cache.num_free_pages() == [64]


def test_decode_tokens_go_first_and_prompts_fill_the_rest():
    cache, sched = make(budget=10)
    a, b = req("a", 6, max_tokens=8), req("b", 30, max_tokens=2)
    sched.add(a)
    run_step(cache, sched)                               # a: whole prompt, first token
    sched.add(b)
    out, _ = run_step(cache, sched)
    assert [(s.request.rid, len(s.tokens)) for s in out.scheduled] == [("a", 1), ("b", 9)]
    out, _ = run_step(cache, sched)
    assert [(s.request.rid, len(s.tokens), s.samples) for s in out.scheduled] == [("a", 1, True), ("b", 9, False)]


def test_stop_on_eos_keeps_the_stop_token_and_minimum_new_tokens_delays_it():
    cache, sched = make()
    a = req("a", 3, max_tokens=10)
    b = req("b", 3, max_tokens=10, minimum_new_tokens=3)
    c = req("c", 3, max_tokens=10, ignore_eos=True, stop_token_ids=(7,))
    for r in (a, b, c):
        sched.add(r)
    script = {"a": [5, 2, 9], "b": [2, 2, 2, 2], "c": [2, 7, 1]}
    while sched.has_work():
        run_step(cache, sched, token_of=lambda r: script[r.rid][len(r.outputs)])
    assert (a.outputs, a.finish_reason) == ([5, 2], "stop")
    assert (b.outputs, b.finish_reason) == ([2, 2, 2], "stop")          # eos counted only from the 3rd token on
    assert (c.outputs, c.finish_reason) == ([2, 7], "stop")
    assert sched.suppressed_ids(req("d", 1, minimum_new_tokens=1)) == [2]


def test_no_more_live_requests_than_sequences_and_fifo_admission():
    cache, sched = make(seqs=2, budget=64)
    rs = [req(f"r{i}", 4, max_tokens=2) for i in range(4)]
    for r in rs:
        sched.add(r)
    out, _ = run_step(cache, sched)
    assert [s.request.rid for s in out.scheduled] == ["r0", "r1"]
    out, finished = run_step(cache, sched)
    assert {r.rid for r in finished} == {"r0", "r1"}
    out, _ = run_step(cache, sched)
    assert [s.request.rid for s in out.scheduled] == ["r2", "r3"]


def test_when_pages_run_out_the_youngest_is_preempted_and_recomputed():
    cache, sched = make(num_pages=6, page_size=4, seqs=3, budget=64)     # 24 tokens of cache
    a, b = req("a", 10, max_tokens=12), req("b", 9, max_tokens=12)
    sched.add(a), sched.add(b)
    preempted = []
    steps = 0
    while sched.has_work():
        out, _ = run_step(cache, sched)
        preempted += [r.rid for r in out.preempted]
        steps += 1
        assert steps < 200
    assert preempted and set(preempted) == {"b"}                           # the younger one goes, never the older
    assert b.preemptions >= 1
    # both finish with all their tokens; the preempted one recomputed prompt + outputs
    assert len(a.outputs) == 12 and len(b.outputs) == 12
    assert a.finish_reason == b.finish_reason == "length"
    assert cache.num_free_pages() == [6]


def test_preemption_does_not_change_what_is_sampled():
    """Sampling is keyed by (seed, ordinal): the scripted sampler here depends on the ordinal only,
    so outputs with and without preemption are the same."""
    outs = []
    for pages in (6, 64):
        cache, sched = make(num_pages=pages, page_size=4, seqs=3, budget=64)
        a, b = req("a", 10, max_tokens=12), req("b", 9, max_tokens=12)
        sched.add(a), sched.add(b)
        while sched.has_work():
            run_step(cache, sched, token_of=lambda r: (hash(r.rid) + 31 * len(r.outputs)) % 1000 + 3)
        outs.append((a.outputs, b.outputs))
    assert outs[0] == outs[1]


def test_a_request_that_can_never_fit_finishes_with_capacity():
    cache, sched = make(num_pages=2, page_size=4, seqs=2, budget=64)       # 8 tokens of cache
    big, small = req("big", 20, max_tokens=2), req("small", 3, max_tokens=2)
    sched.add(big), sched.add(small)
    while sched.has_work():
        run_step(cache, sched)
    assert big.finish_reason == "capacity" and big.outputs == []
    assert small.finish_reason == "length" and len(small.outputs) == 2
    assert cache.num_free_pages() == [2] and cache.slots.num_free == 2


def test_cancel_running_and_waiting():
    cache, sched = make(seqs=1)
    a, b = req("a", 5, max_tokens=5), req("b", 5, max_tokens=5)
    sched.add(a), sched.add(b)
    run_step(cache, sched)
    assert sched.cancel("a").finish_reason == "cancelled" and sched.cancel("b").finish_reason == "cancelled"
    assert not sched.has_work() and cache.num_free_pages() == [64] and sched.cancel("zzz") is None


def test_context_limit_and_empty_prompt_are_refused():
    cache, sched = make(max_context=16)
    with pytest.raises(ValueError, match="context limit"):
        sched.add(req("a", 10, max_tokens=7))
    with pytest.raises(ValueError, match="at least one"):
        sched.add(Request("b", [], SamplingParams()))


def test_sampling_params_follow_the_reference_ranges():
    SamplingParams(temperature=2.0, top_p=0.5, seed=2 ** 63 - 1)
    for bad in (dict(temperature=-0.1), dict(temperature=2.1), dict(top_p=0.0), dict(top_p=1.1),
                dict(temperature=0.0, top_p=0.9), dict(seed=-1), dict(n=2), dict(max_tokens=0),
                dict(temperature=0.0, top_k=5), dict(temperature=1.0, top_k=0), dict(temperature=float("nan"))):
        with pytest.raises(ValueError):
            SamplingParams(**bad)
