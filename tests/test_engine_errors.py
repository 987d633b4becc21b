"""A step whose kernels reported a fault must not count: no token of it is emitted, its requests end with
reason "error" and give everything back, and requests outside it go on as if nothing had happened.

Runs on the CPU with the torch stand-in for the kernels, which reports a key page of -1 in the device's way
(error word 2, no exception).  The fault is made on the host: one block-table entry of one step is overwritten
with -1 on its way into the batch."""
import pytest

from fake_ops import FakeOps
from pih_b200.engine import Engine
from pih_b200.kernels.ops import KernelError
from pih_b200.sampling import SamplingParams
import traces


def _engine(model_dir, run_ahead, **kw):
    args = dict(device="cpu", ops=FakeOps(), page_size=8, max_cache_tokens=1024, maximum_batch_sequences=2,
                maximum_batch_tokens=64, run_ahead=run_ahead)
    args.update(kw)
    return Engine(model_dir, "float32", **args)


def poison_next_block_table(cache):
    """The next block table that is built gets -1 in place of its first request's first page."""
    original = cache.fill_block_table
    state = {"armed": True}

    def fill(g, rids, out):
        original(g, rids, out)
        if state["armed"] and g == 0:
            out[0, 0] = -1
            state["armed"] = False
    cache.fill_block_table = fill
    return state


@pytest.mark.parametrize("run_ahead", [False, True])
def test_a_failed_step_emits_nothing_frees_everything_and_spares_the_others(model_dirs, tiny_configs, run_ahead):
    prompts = list(traces.make_requests(tiny_configs["A"]["vocab_size"], [12, 9, 14, 10], seed=31).values())
    params = SamplingParams(max_tokens=10, ignore_eos=True)
    clean = _engine(model_dirs["A"], run_ahead).complete_batch(prompts, max_tokens=10, ignore_eos=True)

    e = _engine(model_dirs["A"], run_ahead)
    reqs = [e._live[e.submit(p, params)] for p in prompts[:3]]       # two run, the third waits for a slot
    for _ in range(4):
        e.step()
    assert [r.status for r in reqs] == ["running", "running", "waiting"]
    before = [list(r.outputs) for r in reqs]
    armed = poison_next_block_table(e.cache)
    with pytest.raises(KernelError, match="maps to no cache page"):
        for _ in range(4):
            e.step()
    assert not armed["armed"]
    # the two requests of the failed step: ended with "error", at most the tokens of steps seen to succeed —
    # all of them tokens of the clean run — and nothing more is ever added
    for r, c in zip(reqs[:2], clean[:2]):
        assert r.status == "finished" and r.finish_reason == "error"
        assert r.outputs == c["token_ids"][:len(r.outputs)] and len(r.outputs) < 10
    assert len(reqs[0].outputs) <= len(before[0]) + 1
    assert int(e.rt.ops.error_word) == 0                            # cleared for the steps that follow
    e.cache.check()
    assert e.cache.slots.num_free == 2
    assert all(f == e.cache.num_pages for f in e.cache.num_free_pages())
    # the request that was waiting, and one that arrives afterwards, run as in an engine without the fault
    late = e._live[e.submit(prompts[3], params)]
    while e.has_work():
        e.step()
    assert reqs[2].outputs == clean[2]["token_ids"] and reqs[2].finish_reason == "length"
    assert late.outputs == clean[3]["token_ids"]
    e.cache.check()
    assert all(f == e.cache.num_pages for f in e.cache.num_free_pages())


def test_complete_batch_leaves_nothing_behind_after_a_fault(model_dirs, tiny_configs):
    prompts = list(traces.make_requests(tiny_configs["B"]["vocab_size"], [20, 5, 9], seed=32).values())
    e = _engine(model_dirs["B"], True, maximum_batch_sequences=4)
    want = e.complete_batch(prompts, max_tokens=6, ignore_eos=True)
    poison_next_block_table(e.cache)
    with pytest.raises(KernelError):
        e.complete_batch(prompts, max_tokens=6, ignore_eos=True)
    assert not e.has_work() and not e._live
    e.cache.check()
    assert all(f == e.cache.num_pages for f in e.cache.num_free_pages())
    assert e.complete_batch(prompts, max_tokens=6, ignore_eos=True) == want


def test_a_fault_in_a_prompt_portion_is_seen_before_any_token_is_emitted(model_dirs, tiny_configs):
    """The portion steps sample nothing, so nobody waits for them; their error word is looked at when the
    first sampling step is collected, before its token is booked."""
    prompt = traces.make_requests(tiny_configs["A"]["vocab_size"], [40], seed=33)["r0"]
    e = _engine(model_dirs["A"], True, maximum_batch_tokens=16)
    req = e._live[e.submit(prompt, SamplingParams(max_tokens=4, ignore_eos=True))]
    e.step()                                           # first portion
    poison_next_block_table(e.cache)                   # second portion reads the first one's keys
    with pytest.raises(KernelError):
        for _ in range(4):
            e.step()
    assert req.outputs == [] and req.finish_reason == "error"
    assert all(f == e.cache.num_pages for f in e.cache.num_free_pages())
