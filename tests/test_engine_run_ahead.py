"""Planning the next decode step while the current one runs must not change a single token.

Runs the engine on the CPU with the torch stand-in for the kernels: the same requests with and without
run-ahead — different lengths, a stop token in the middle of a generation, temperature sampling, a request
that arrives late, one that is cancelled, and a pool so small that requests are preempted."""
import pytest

from fake_ops import FakeOps
from pih_b200.engine import Engine
from pih_b200.sampling import SamplingParams
import traces


def _engine(model_dir, run_ahead, **kw):
    args = dict(device="cpu", ops=FakeOps(), page_size=8, max_cache_tokens=1024, maximum_batch_sequences=4,
                maximum_batch_tokens=16, run_ahead=run_ahead)
    args.update(kw)
    return Engine(model_dir, "float32", **args)


def _prompts(vocab, lengths, seed):
    return list(traces.make_requests(vocab, lengths, seed=seed).values())


@pytest.mark.parametrize("temperature", [0.0, 0.8])
def test_run_ahead_gives_the_same_tokens(model_dirs, tiny_configs, temperature):
    prompts = _prompts(tiny_configs["B"]["vocab_size"], [3, 20, 9, 33], seed=5)
    per_prompt = [dict(max_tokens=m) for m in (14, 5, 9, 1)]
    kw = dict(temperature=temperature, seed=3, ignore_eos=True, parameters_per_prompt=per_prompt)
    plain = _engine(model_dirs["B"], False)
    ahead = _engine(model_dirs["B"], True)
    want = plain.complete_batch(prompts, **kw)
    got = ahead.complete_batch(prompts, **kw)
    assert got == want
    assert plain.steps_planned_ahead == 0 and ahead.steps_planned_ahead >= 5
    for e in (plain, ahead):
        e.cache.check()
        assert all(f == e.cache.num_pages for f in e.cache.num_free_pages())
        assert not e.has_work()


def test_a_stop_token_found_late_drops_the_token_computed_ahead(model_dirs, tiny_configs):
    prompts = _prompts(tiny_configs["A"]["vocab_size"], [12, 7], seed=8)
    free = _engine(model_dirs["A"], False, page_size=16).complete_batch(prompts, max_tokens=12, ignore_eos=True)
    stop = free[0]["token_ids"][5]                     # the first request produces this id as its sixth token at the latest
    kw = dict(max_tokens=12, ignore_eos=True, stop_token_ids=[stop])
    want = _engine(model_dirs["A"], False, page_size=16).complete_batch(prompts, **kw)
    ahead = _engine(model_dirs["A"], True, page_size=16)
    got = ahead.complete_batch(prompts, **kw)
    assert got == want and want[0]["finish_reason"] == "stop" and len(want[0]["token_ids"]) <= 6
    assert ahead.steps_planned_ahead > 0
    ahead.cache.check()
    assert all(f == ahead.cache.num_pages for f in ahead.cache.num_free_pages())


def test_run_ahead_with_late_arrival_cancel_and_preemption(model_dirs, tiny_configs):
    vocab = tiny_configs["B"]["vocab_size"]
    prompts = _prompts(vocab, [30, 25, 28, 6], seed=13)

    def run(run_ahead):
        # 16 pages of 8: the three long requests (8 + 7 + 8 pages at their ends) do not fit together
        e = _engine(model_dirs["B"], run_ahead, max_cache_tokens=128, maximum_batch_tokens=32)
        reqs = [e._live[e.submit(p, SamplingParams(max_tokens=30, ignore_eos=True))] for p in prompts[:3]]
        steps = 0
        late = victim = None
        while e.has_work():
            e.step()
            steps += 1
            if steps == 4:
                late = e._live[e.submit(prompts[3], SamplingParams(max_tokens=6, ignore_eos=True))]
            if steps == 16:
                victim = reqs[1]
                e.cancel(victim.rid)
        e.cache.check()
        assert all(f == e.cache.num_pages for f in e.cache.num_free_pages())
        outs = [(r.outputs if r is not victim else None, r.finish_reason) for r in reqs + [late]]
        return outs, sum(r.preemptions for r in reqs + [late]), e.steps_planned_ahead

    want, preempted, _ = run(False)
    got, preempted_ahead, planned = run(True)
    assert preempted > 0 and planned > 0
    assert got == want


def test_an_engine_around_a_model_that_is_already_built(model_dirs, tiny_configs):
    """``Engine(model=(configuration, model))`` gives the tokens of the engine that loads the folder itself."""
    import torch
    from pih_b200.models import load_model
    from pih_b200.parts import Runtime
    prompts = _prompts(tiny_configs["A"]["vocab_size"], [5, 11, 17], seed=2)
    want = _engine(model_dirs["A"], True, page_size=16).complete_batch(prompts, max_tokens=8, ignore_eos=True)
    rt = Runtime(torch.device("cpu"), torch.float32, FakeOps())
    config, model = load_model(model_dirs["A"], rt)
    built = Engine("tiny-a", model=(config, model), page_size=16, max_cache_tokens=1024, maximum_batch_sequences=4,
                   maximum_batch_tokens=16)
    assert built.complete_batch(prompts, max_tokens=8, ignore_eos=True) == want
    assert built.models()["data"][0]["id"] == "tiny-a"


@pytest.mark.parametrize("seed", range(6))
def test_random_workloads_give_the_same_tokens_with_and_without_run_ahead(model_dirs, tiny_configs, seed):
    """Seeded random workloads — arrivals over time, lengths, limits, temperatures, a stop id, cancellations, a pool
    that forces preemptions in some of them: after every step the cache's books are right and no step holds
    more tokens or requests than allowed; at the end every page is free; and planning ahead changes no token."""
    import random
    name = "AB"[seed % 2]
    vocab = tiny_configs[name]["vocab_size"]
    rng = random.Random(100 + seed)
    n = rng.randint(4, 7)
    lengths = [rng.randint(1, 40) for _ in range(n)]
    prompts = _prompts(vocab, lengths, seed=seed)
    arrive = sorted(rng.randint(0, 12) for _ in range(n))
    limits = [rng.randint(1, 20) for _ in range(n)]
    temps = [rng.choice([0.0, 0.0, 0.7]) for _ in range(n)]
    stop_id = rng.randrange(vocab)
    cancel_at = {rng.randint(3, 25): rng.randrange(n) for _ in range(rng.randint(0, 2))}
    budget, seqs = rng.choice([8, 16, 32]), rng.choice([2, 3, 4])
    pool_tokens = rng.choice([96, 160, 1024])
    longest = max(a + b for a, b in zip(lengths, limits))
    pool_tokens = max(pool_tokens, -(-longest // 8) * 8 + 8)       # the longest request fits alone

    def run(run_ahead):
        e = _engine(model_dirs[name], run_ahead, max_cache_tokens=pool_tokens, maximum_batch_tokens=budget,
                    maximum_batch_sequences=seqs)
        reqs, cancelled = {}, set()
        step = 0
        while step < 400 and (e.has_work() or len(reqs) < n):
            for i in range(n):
                if i not in reqs and arrive[i] <= step:
                    params = SamplingParams(max_tokens=limits[i], temperature=temps[i], seed=seed + i,
                                            stop_token_ids=(stop_id,), ignore_eos=True)
                    reqs[i] = e._live[e.submit(prompts[i], params)]
            if step in cancel_at and cancel_at[step] in reqs and reqs[cancel_at[step]].status != "finished":
                cancelled.add(cancel_at[step])
                e.cancel(reqs[cancel_at[step]].rid)
            if e.has_work():
                e.step()
            e.cache.check()
            step += 1
        assert not e.has_work() and len(reqs) == n
        assert all(f == e.cache.num_pages for f in e.cache.num_free_pages())
        for i, r in reqs.items():
            if i not in cancelled:
                assert r.status == "finished" and 1 <= len(r.outputs) <= limits[i]
                if r.finish_reason == "stop":
                    assert r.outputs[-1] == stop_id and stop_id not in r.outputs[:-1]
                else:
                    assert r.finish_reason == "length" and len(r.outputs) == limits[i]
        return {i: (r.outputs, r.finish_reason) for i, r in reqs.items() if i not in cancelled}

    assert run(True) == run(False)


@pytest.mark.parametrize("temperature", [0.0, 0.9])
def test_log_probabilities_come_back_with_the_tokens(model_dirs, tiny_configs, temperature):
    """``logprobs=True``: one log-probability per generated token (the reference's selected_logprob), the same
    with and without a step planned ahead, equal to the plain implementation's log-softmax of the scaled logits at
    the token; a request that did not ask gets none."""
    import plain_impl
    import torch
    from conftest import load_plain_weights
    prompts = _prompts(tiny_configs["A"]["vocab_size"], [11, 4], seed=9)
    per_prompt = [dict(logprobs=True), dict()]
    kw = dict(max_tokens=7, temperature=temperature, seed=4, ignore_eos=True, parameters_per_prompt=per_prompt)
    got = _engine(model_dirs["A"], True, page_size=16).complete_batch(prompts, **kw)
    assert got == _engine(model_dirs["A"], False, page_size=16).complete_batch(prompts, **kw)
    assert "logprobs" not in got[1] and len(got[0]["logprobs"]) == 7
    cfg, w = load_plain_weights(model_dirs["A"])
    tokens = prompts[0] + got[0]["token_ids"]
    logits = plain_impl.forward(cfg, w, tokens)[len(prompts[0]) - 1:-1]
    scaled = logits.double() / (temperature if temperature > 0 else 1.0)
    want = torch.log_softmax(scaled, dim=-1)[torch.arange(7), torch.tensor(got[0]["token_ids"])]
    torch.testing.assert_close(torch.tensor(got[0]["logprobs"], dtype=torch.float64), want, rtol=1e-4, atol=1e-4)


def test_the_most_probable_ids_come_back_with_the_tokens(model_dirs, tiny_configs):
    """``top_logprobs=n`` (with ``logprobs``): per generated token the n most probable ids with their
    log-probabilities, best first — the plain implementation's ordering of the scaled logits; each request gets as
    many as it asked for, one that did not ask gets none; and the option needs ``logprobs`` and stays within 20."""
    import plain_impl
    from conftest import load_plain_weights
    from pih_b200.sampling import SamplingParams
    prompts = _prompts(tiny_configs["A"]["vocab_size"], [9, 5, 6], seed=10)
    per_prompt = [dict(logprobs=True, top_logprobs=5), dict(logprobs=True, top_logprobs=2, temperature=0.7, seed=2),
                  dict(logprobs=True)]
    kw = dict(max_tokens=6, ignore_eos=True, parameters_per_prompt=per_prompt)
    got = _engine(model_dirs["A"], True, page_size=16).complete_batch(prompts, **kw)
    assert got == _engine(model_dirs["A"], False, page_size=16).complete_batch(prompts, **kw)
    assert "top_logprobs" not in got[2]
    cfg, w = load_plain_weights(model_dirs["A"])
    for r, prompt, n, temperature in ((got[0], prompts[0], 5, 0.0), (got[1], prompts[1], 2, 0.7)):
        assert len(r["top_logprobs"]) == 6
        logits = plain_impl.forward(cfg, w, prompt + r["token_ids"])[len(prompt) - 1:-1]
        for step, row in enumerate(r["top_logprobs"]):
            want = plain_impl.top_logprobs(logits[step].tolist(), n, temperature=temperature)
            assert [e["token_id"] for e in row] == [i for i, _ in want]
            assert all(abs(e["logprob"] - lp) < 1e-4 for e, (_, lp) in zip(row, want))
            if temperature == 0.0:                              # greedy: the first of them is the token, with its logprob
                assert row[0]["token_id"] == r["token_ids"][step]
                assert abs(row[0]["logprob"] - r["logprobs"][step]) < 1e-5
    with pytest.raises(ValueError):
        SamplingParams(top_logprobs=3)
    with pytest.raises(ValueError):
        SamplingParams(logprobs=True, top_logprobs=21)
    # more ids than the vocabulary leaves beside those that may be suppressed: refused when the request is handed in
    tiny = _engine(model_dirs["A"], False, page_size=16)
    import dataclasses
    tiny.model.spec = dataclasses.replace(tiny.model.spec, vocab=12)       # (only what submit looks at)
    with pytest.raises(ValueError, match="top_logprobs"):
        tiny.submit([1, 2, 3], SamplingParams(logprobs=True, top_logprobs=12))
    assert not tiny.has_work()

