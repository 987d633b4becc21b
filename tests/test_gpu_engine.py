"""The serving loop on the GPU in the schedules that small pools, faults and stand-in requests bring about:
preemption and recomputation with CUDA graphs and run-ahead, a step whose kernels report a fault, and the
default pool size."""
import random

import pytest
import torch

import plain_impl
import traces
from conftest import load_plain_weights

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _prompts(vocab, lengths, seed):
    return list(traces.make_requests(vocab, lengths, seed=seed).values())


def _engine(model_dir, dtype="float32", **kw):
    from pih_b200.engine import Engine
    # (graphs at the first sight of a decode shape: these short runs are here to exercise them)
    args = dict(page_size=8, max_cache_tokens=1024, maximum_batch_sequences=4, maximum_batch_tokens=32,
                capture_decode_after=0)
    args.update(kw)
    return Engine(model_dir, dtype, **args)


def _all_back(e):
    e.drain()
    e.rt.ops.check_errors()
    e.cache.check()
    assert all(f == e.cache.num_pages for f in e.cache.num_free_pages())
    assert e.cache.slots.num_free == e.cache.max_requests and not e.has_work()


@pytest.mark.parametrize("temperature", [0.0, 0.8])
@pytest.mark.parametrize("run_ahead", [False, True])
def test_preempted_requests_are_recomputed_to_the_same_tokens(model_dirs, tiny_configs, run_ahead, temperature):
    """A pool of 16 pages of 8 for three requests that need 8 + 7 + 8 at their ends, and a fourth that arrives
    later: requests are preempted, their pages go to others in the same step, and they are computed again —
    with CUDA graphs on, with and without a step queued ahead.  The tokens are those of an engine whose pool
    never runs out, and, when greedy, those of the plain implementation."""
    from pih_b200.sampling import SamplingParams
    vocab = tiny_configs["B"]["vocab_size"]
    prompts = _prompts(vocab, [30, 25, 28, 6], seed=13)
    params = SamplingParams(max_tokens=30, temperature=temperature, seed=5, ignore_eos=True)

    def run(pool_tokens):
        e = _engine(model_dirs["B"], max_cache_tokens=pool_tokens, run_ahead=run_ahead, cuda_graphs=True)
        reqs = [e._live[e.submit(p, params)] for p in prompts[:3]]
        steps = 0
        while e.has_work():
            e.step()
            e.cache.check()
            steps += 1
            if steps == 4:
                reqs.append(e._live[e.submit(prompts[3], SamplingParams(max_tokens=6, temperature=temperature,
                                                                         seed=6, ignore_eos=True))])
        _all_back(e)
        return [r.outputs for r in reqs], sum(r.preemptions for r in reqs), e.steps_planned_ahead

    want, none_preempted, _ = run(1024)
    got, preempted, planned = run(128)
    assert none_preempted == 0 and preempted >= 2
    assert (planned > 0) == run_ahead
    assert got == want
    if temperature == 0.0:
        cfg, w = load_plain_weights(model_dirs["B"])
        for prompt, tokens in zip(prompts, got):
            assert tokens == plain_impl.generate_greedy(cfg, w, prompt, len(tokens))


@pytest.mark.parametrize("seed", range(4))
def test_random_workloads_on_the_gpu(model_dirs, tiny_configs, seed):
    """Seeded random workloads (arrivals over time, limits, temperatures, a stop id, cancellations, pools that
    force preemptions in some): run-ahead changes no token, the books are right after every step, every page
    comes back."""
    from pih_b200.sampling import SamplingParams
    name = "AB"[seed % 2]
    vocab = tiny_configs[name]["vocab_size"]
    rng = random.Random(200 + seed)
    n = rng.randint(4, 7)
    lengths = [rng.randint(1, 40) for _ in range(n)]
    prompts = _prompts(vocab, lengths, seed=seed)
    arrive = sorted(rng.randint(0, 12) for _ in range(n))
    limits = [rng.randint(1, 20) for _ in range(n)]
    temps = [rng.choice([0.0, 0.0, 0.7]) for _ in range(n)]
    stop_id = rng.randrange(vocab)
    cancel_at = {rng.randint(3, 25): rng.randrange(n) for _ in range(rng.randint(0, 2))}
    budget, seqs = rng.choice([8, 16, 32]), rng.choice([2, 3, 4])
    longest = max(a + b for a, b in zip(lengths, limits))
    pool_tokens = max(rng.choice([96, 160, 1024]), -(-longest // 8) * 8 + 8)

    def run(run_ahead):
        e = _engine(model_dirs[name], max_cache_tokens=pool_tokens, maximum_batch_tokens=budget,
                    maximum_batch_sequences=seqs, run_ahead=run_ahead, cuda_graphs=True)
        reqs, cancelled = {}, set()
        step = 0
        while step < 400 and (e.has_work() or len(reqs) < n):
            for i in range(n):
                if i not in reqs and arrive[i] <= step:
                    reqs[i] = e._live[e.submit(prompts[i], SamplingParams(
                        max_tokens=limits[i], temperature=temps[i], seed=seed + i, stop_token_ids=(stop_id,),
                        ignore_eos=True))]
            if step in cancel_at and cancel_at[step] in reqs and reqs[cancel_at[step]].status != "finished":
                cancelled.add(cancel_at[step])
                e.cancel(reqs[cancel_at[step]].rid)
            if e.has_work():
                e.step()
            e.cache.check()
            step += 1
        assert len(reqs) == n
        _all_back(e)
        return {i: (r.outputs, r.finish_reason) for i, r in reqs.items() if i not in cancelled}

    assert run(True) == run(False)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("run_ahead", [False, True])
def test_a_step_that_reports_a_fault_does_not_count(model_dirs, tiny_configs, run_ahead, dtype):
    """One block-table entry of one decode step is overwritten with -1 on the host, so the attention kernel
    finds a visible key without a page and reports it in the error word — no trap, no exception on the
    device.  The engine sees the word with the step's ids: the step's requests end with reason "error", no
    token of it is emitted, every page comes back, and the requests outside the step go on unharmed."""
    from pih_b200.kernels.ops import KernelError
    from pih_b200.sampling import SamplingParams
    name = "C" if dtype == "bfloat16" else "A"              # C: head size 64, the TMA-fed decode kernel
    page = 16
    prompts = _prompts(tiny_configs[name]["vocab_size"], [12, 9, 14, 10], seed=31)
    params = SamplingParams(max_tokens=10, ignore_eos=True)
    kw = dict(page_size=page, maximum_batch_sequences=2, maximum_batch_tokens=64, run_ahead=run_ahead, cuda_graphs=True)
    clean = _engine(model_dirs[name], dtype, **kw).complete_batch(prompts, max_tokens=10, ignore_eos=True)

    e = _engine(model_dirs[name], dtype, **kw)
    reqs = [e._live[e.submit(p, params)] for p in prompts[:3]]       # two run, the third waits for a slot
    for _ in range(4):
        e.step()
    assert [r.status for r in reqs] == ["running", "running", "waiting"]
    before = len(reqs[0].outputs)
    original = e.cache.fill_block_table
    armed = [True]

    def poisoned(g, rids, out):
        original(g, rids, out)
        if armed[0] and g == 0:
            out[0, 0] = -1
            armed[0] = False
    e.cache.fill_block_table = poisoned
    with pytest.raises(KernelError, match="maps to no cache page"):
        for _ in range(4):
            e.step()
    assert not armed[0]
    for r, c in zip(reqs[:2], clean[:2]):
        assert r.status == "finished" and r.finish_reason == "error"
        assert r.outputs == c["token_ids"][:len(r.outputs)] and len(r.outputs) <= before + 1
    torch.cuda.synchronize()
    assert int(e.rt.ops.error_word.item()) == 0
    e.cache.check()
    assert all(f == e.cache.num_pages for f in e.cache.num_free_pages()) and e.cache.slots.num_free == 2
    late = e._live[e.submit(prompts[3], params)]
    while e.has_work():
        e.step()
    assert reqs[2].outputs == clean[2]["token_ids"] and late.outputs == clean[3]["token_ids"]
    _all_back(e)


def test_the_default_pool_comes_from_the_devices_memory(model_dirs, tiny_configs):
    from pih_b200.engine import Engine
    e = Engine(model_dirs["A"], "bfloat16", maximum_batch_sequences=8)
    assert e.cache_tokens == 8 * tiny_configs["A"]["max_position_embeddings"]       # plenty of memory: the cap
    prompts = _prompts(tiny_configs["A"]["vocab_size"], [5, 11], seed=3)
    got = e.complete_batch(prompts, max_tokens=4, ignore_eos=True)
    assert [len(r["token_ids"]) for r in got] == [4, 4]
    with pytest.raises(MemoryError, match="fewer than one request"):
        Engine(model_dirs["A"], "bfloat16", memory_fraction=1e-6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_warm_up_captures_shapes_and_leaves_nothing_behind(model_dirs, tiny_configs, dtype):
    """Before the first request the engine runs and captures the shapes that its limits make likely, with stand-in
    requests; afterwards the pool is whole, and requests are answered with the tokens of an engine that was
    not warmed up — now from graphs captured beforehand, padded to the shapes of the warm-up."""
    vocab = tiny_configs["A"]["vocab_size"]
    prompts = _prompts(vocab, [45, 9, 70, 23, 31], seed=17)

    def run(warm):
        e = _engine(model_dirs["A"], dtype, page_size=16, max_cache_tokens=2048, maximum_batch_sequences=6,
                    maximum_batch_tokens=48, cuda_graphs=True, capture_decode_after=2)
        done = e.warm_up() if warm else None
        if warm:
            assert done["decode_batches"] == [1, 2, 3, 4, 5, 6] and done["graphs"] >= 6 + 4, done
            assert ("stopped" not in done) and not e.cache.requests
            assert all(f == e.cache.num_pages for f in e.cache.num_free_pages())
        before = len(e.runner._graphs)
        got = e.complete_batch(prompts, max_tokens=12, ignore_eos=True)
        _all_back(e)
        return [r["token_ids"] for r in got], before, len(e.runner._graphs)

    cold, _, _ = run(False)
    warm, before, after = run(True)
    assert warm == cold
    assert after - before <= 4, "most shapes of the run should have been captured by the warm-up"
    with pytest.raises(RuntimeError, match="without requests"):
        e = _engine(model_dirs["A"], dtype, cuda_graphs=True)
        e.submit(prompts[0])
        e.warm_up()
