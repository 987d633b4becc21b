"""The engine on the GPU against the plain implementation, in 32-bit and in
bfloat16, for every way of cutting the same requests into steps: whole; most
in one step and the last 32 tokens one by one; portions of changing size down
to two tokens; mixed batches of up to four live requests with so few pages
that they are used again.  Also through ``bin/trace_run`` as a user runs it."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_impl
import traces
from conftest import ROOT, load_plain_weights

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [70, 45, 90, 33, 61, 50, 77, 40], "B": [64, 33, 97, 41, 80, 55, 35, 66],
           "C": [130, 45, 257, 64, 33, 150, 65, 90], "D": [129, 40, 200, 64, 35, 70, 128, 50]}
PAGE = {"A": 16, "B": 8, "C": 16, "D": 32}
FAMILIES = ["whole", "tail_decode", "portions", "mixed"]

# 32-bit: accumulation-order noise only (logits are O(1)).
TOL_F32 = 2e-5
# bfloat16: every op rounds its output to 8 bits of mantissa, so even the plain implementation with
# the reference's rounding places ("plain-bf16") sits a measurable distance from the unrounded truth,
# and any two bf16 implementations that differ in one accumulation order decorrelate from each other
# by about that distance.  The yardstick is therefore measured, per request, inside the test:
# E = |plain-bf16 - truth|.  The engine must be as close to the truth as plain-bf16 is, within half
# again (mean and worst position), and within the triangle's reach of plain-bf16 itself.
BF16_TRUTH_FACTOR, BF16_PLAIN_FACTOR, BF16_FLOOR = 1.5, 2.5, 0.004

_REF = {}


def reference(model_dir, name, requests, rounding):
    key = (name, rounding)
    if key not in _REF:
        cfg, w = load_plain_weights(model_dir)
        _REF[key] = {rid: plain_impl.forward(cfg, w, toks, rounding) for rid, toks in requests.items()}
    return _REF[key]


def compare(got, truth, dtype, what, plain_bf16=None):
    for rid in truth:
        g, r = got[rid].double(), truth[rid]
        assert g.shape == r.shape, (what, rid, g.shape, r.shape)
        err = (g - r).abs()
        if dtype == "float32":
            worst = int(err.max(dim=1).values.argmax())
            assert float(err.max()) < TOL_F32, f"{what} {rid}: max abs error {float(err.max()):.3e} at position {worst}"
            continue
        spread = float(r.std())
        yard = (plain_bf16[rid] - r).abs()
        worst = int(err.max(dim=1).values.argmax())
        assert float(err.mean()) <= BF16_TRUTH_FACTOR * float(yard.mean()), \
            f"{what} {rid}: mean error {float(err.mean()):.5f} vs plain-bf16's own {float(yard.mean()):.5f}"
        assert float(err.max()) <= BF16_TRUTH_FACTOR * float(yard.max()) + BF16_FLOOR * spread, \
            f"{what} {rid}: worst error {float(err.max()):.5f} at position {worst} vs plain-bf16's own {float(yard.max()):.5f}"
        apart = (g - plain_bf16[rid]).abs()
        assert float(apart.mean()) <= BF16_PLAIN_FACTOR * float(yard.mean()), (what, rid, float(apart.mean()))
        assert float(apart.max()) <= BF16_PLAIN_FACTOR * float(yard.max()) + BF16_FLOOR * spread, \
            (what, rid, float(apart.max()))


def compare_with_plain(got, model_dir, name, requests, dtype, what):
    truth = reference(model_dir, name, requests, "none")
    plain = reference(model_dir, name, requests, "bf16") if dtype == "bfloat16" else None
    compare(got, truth, dtype, what, plain)


@pytest.fixture(scope="module")
def requests_of(tiny_configs):
    return {n: traces.make_requests(tiny_configs[n]["vocab_size"], LENGTHS[n], seed=11) for n in ("A", "B", "C", "D")}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("family", FAMILIES)
def test_replay_families(model_dirs, requests_of, name, dtype, family):
    from pih_b200.engine.factory import create_runner
    requests = requests_of[name]
    steps = getattr(traces, family)(requests)
    pool = traces.peak_tokens(steps, round_to=64)
    _, model, cache, runner = create_runner(model_dirs[name], dtype, page_size=PAGE[name],
                                            max_cache_tokens=pool, max_requests=4)
    got = traces.replay(runner, steps)
    model.rt.ops.check_errors()
    compare_with_plain(got, model_dirs[name], name, requests, dtype, f"{name} {family}")
    cache.check()
    assert all(f == cache.num_pages for f in cache.num_free_pages())
    if family == "mixed":
        assert all(g.pool.pages_handed_out > g.pool.num_pages for g in cache.groups)


@pytest.mark.parametrize("name", ["A", "C", "D"])
@pytest.mark.parametrize("family", ["whole", "mixed"])
def test_replay_with_the_gate_up_product_on_pairs_of_sms(model_dirs, tiny_configs, requests_of, name, family):
    """The gate/up product of large prompt portions runs on the pack's tcgen05 kernel on pairs of SMs with SiLU-mul
    in its epilogue; the tiny models' steps never reach its row count.  With the rule opened to every step of more
    than 16 rows, whole prompts and mixed steps still agree with the plain implementation."""
    from pih_b200.engine.factory import create_runner
    requests = requests_of[name]
    steps = getattr(traces, family)(requests)
    _, model, cache, runner = create_runner(model_dirs[name], "bfloat16", page_size=PAGE[name],
                                            max_cache_tokens=traces.peak_tokens(steps, round_to=64), max_requests=4)
    ops = model.rt.ops
    rows = ops.tcgen05_swiglu_min_rows
    ops.set_pair_swiglu_rule(17, 0)
    try:
        assert ops.lib.pih_pair_swiglu_wanted(17, 2 * tiny_configs[name]["intermediate_size"]) == 1
        got = traces.replay(runner, steps)
        ops.check_errors()
    finally:
        ops.set_pair_swiglu_rule(rows, 80)
    compare_with_plain(got, model_dirs[name], name, requests, "bfloat16", f"{name} {family} on pairs")
    cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_32bit_and_bf16_cuttings_agree_with_each_other(model_dirs, requests_of, dtype):
    """Beyond the plain implementation: the engine's own cuttings agree among themselves.
    In 32-bit every reduction has a fixed order, so they agree to the last bits."""
    from pih_b200.engine.factory import create_runner
    name = "B"
    requests = requests_of[name]
    outs = {}
    for family in FAMILIES:
        steps = getattr(traces, family)(requests)
        _, _, _, runner = create_runner(model_dirs[name], dtype, page_size=PAGE[name],
                                        max_cache_tokens=traces.peak_tokens(steps), max_requests=4)
        outs[family] = traces.replay(runner, steps)
    for family in FAMILIES[1:]:
        for rid in requests:
            diff = float((outs[family][rid] - outs["whole"][rid]).abs().max())
            # bf16: different kernels serve different cuttings (tile, split, graph); they may differ by rounding
            bound = 1e-6 if dtype == "float32" else 0.08 * float(outs["whole"][rid].std())
            assert diff <= bound, (family, rid, diff)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_replayed_from_cuda_graphs_match(model_dirs, tiny_configs, dtype):
    """Prompt portions of a repeated size and decode steps are captured into CUDA graphs and replayed with
    other requests' data: first sight (as it is), second (capture) and third (replay) all match the plain
    implementation, also when the replayed request starts deep in its context."""
    from pih_b200.engine import StepEntry
    from pih_b200.engine.factory import create_runner
    name = "A"
    reqs = traces.make_requests(tiny_configs[name]["vocab_size"], [300, 300, 300, 428], seed=31)
    _, model, cache, runner = create_runner(model_dirs[name], dtype, page_size=16, max_cache_tokens=1024,
                                            max_requests=4, cuda_graphs=True)
    got = {}
    for rid, toks in reqs.items():
        lead = len(toks) - 300                     # r3 first brings 128 rows (another shape), then 300 like the others
        rows = []
        if lead:
            rows.append(runner.step([StepEntry(rid, toks[:lead], [lead - 1])]).float().cpu())
        rows.append(runner.step([StepEntry(rid, toks[lead:lead + 172], [171])]).float().cpu())   # 172 rows, last wanted
        rows.append(runner.step([StepEntry(rid, toks[lead + 172:], [127])]).float().cpu())       # 128 rows, last wanted
        got[rid] = torch.cat(rows)
        runner.finish(rid)
    model.rt.ops.check_errors()
    assert any(k[0] in ("step", "padded") for k in runner._graphs), "no prompt portion was replayed from a graph"
    cfg, w = load_plain_weights(model_dirs[name])
    for rid, toks in reqs.items():
        lead = len(toks) - 300
        places = ([lead - 1] if lead else []) + [lead + 171, len(toks) - 1]
        truth = plain_impl.forward(cfg, w, toks)[places]
        plain = plain_impl.forward(cfg, w, toks, "bf16")[places] if dtype == "bfloat16" else None
        compare({rid: got[rid]}, {rid: truth}, dtype, f"graph {rid}", {rid: plain} if plain is not None else None)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_mixed_steps_replayed_from_cuda_graphs_match(model_dirs, tiny_configs, name, dtype):
    """Steps that hold decode tokens of two requests beside a prompt portion of a third repeat their shape
    (chunked prefill under a token budget does): the second sighting is captured, later ones are replayed
    with other requests in the rows — every logit still matches the plain implementation."""
    from pih_b200.engine import StepEntry
    from pih_b200.engine.factory import create_runner
    vocab = tiny_configs[name]["vocab_size"]
    decoders = traces.make_requests(vocab, [60, 45], seed=41)                       # d0, d1: 20 decode steps each
    arrivals = {f"p{i}": t for i, t in enumerate(traces.make_requests(vocab, [260] * 4, seed=42).values())}
    _, model, cache, runner = create_runner(model_dirs[name], dtype, page_size=PAGE[name],
                                            max_cache_tokens=1536, max_requests=4, cuda_graphs=True)
    got = {rid: [] for rid in list(decoders) + list(arrivals)}
    places = {rid: [] for rid in got}
    lead = {rid: len(t) - 8 for rid, t in decoders.items()}
    for rid, toks in decoders.items():                                                # prompts, whole
        got[rid].append(runner.step([StepEntry(rid, toks[:lead[rid]], [lead[rid] - 1])]).float().cpu())
        places[rid].append(lead[rid] - 1)
    fed = dict(lead)
    for i, (rid, toks) in enumerate(arrivals.items()):
        for lo in (0, 130):                                                           # two portions of 130 rows
            entries = []
            for d, dt in decoders.items():
                entries.append(StepEntry(d, [dt[fed[d]]], [0]))
            entries.append(StepEntry(rid, toks[lo:lo + 130], [129] if lo else []))
            out = runner.step(entries).float().cpu()
            for k, d in enumerate(decoders):
                got[d].append(out[k:k + 1])
                places[d].append(fed[d])
                fed[d] += 1
            if lo:
                got[rid].append(out[len(decoders):])
                places[rid].append(259)
        runner.finish(rid)
    model.rt.ops.check_errors()
    assert any(k[0] == "padded" or (k[0] == "step" and len(k[1]) == 3) for k in runner._graphs), \
        "no mixed step was replayed from a graph"
    cfg, w = load_plain_weights(model_dirs[name])
    for rid, toks in {**decoders, **arrivals}.items():
        truth = plain_impl.forward(cfg, w, toks)[places[rid]]
        plain = plain_impl.forward(cfg, w, toks, "bf16")[places[rid]] if dtype == "bfloat16" else None
        compare({rid: torch.cat(got[rid])}, {rid: truth}, dtype, f"mixed graph {rid}", {rid: plain} if plain is not None else None)
    cache.check()


def _run_trace_run(model_dir, dtype, steps, out_dir, max_tokens, env=None):
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens)]
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [ln for ln in proc.stdout.splitlines() if ln.startswith("done ")] == [f"done {s['step']}" for s in steps]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(model_dirs, requests_of, tmp_path, dtype):
    """bin/trace_run with its default page size, mixed trace, pool = the peak of live tokens."""
    name = "B"
    requests = requests_of[name]
    steps = traces.mixed(requests, seed=3)
    out_dir = str(tmp_path / "out")
    _run_trace_run(model_dirs[name], dtype, steps, out_dir, traces.peak_tokens(steps))
    cfg, _ = load_plain_weights(model_dirs[name])
    rows = {}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        data = np.fromfile(os.path.join(out_dir, f"{s['step']}.f32"), dtype="<f4").reshape(wanted, cfg["vocab_size"])
        i = 0
        for e in s["entries"]:
            for _ in e["want"]:
                rows.setdefault(e["id"], []).append(torch.from_numpy(data[i].copy()))
                i += 1
    got = {rid: torch.stack(v) for rid, v in rows.items()}
    compare_with_plain(got, model_dirs[name], name, requests, dtype, f"trace_run {dtype}")


def test_trace_run_steps_without_wanted_logits_and_pauses(model_dirs, tmp_path):
    """A step may want nothing (no file is written) and a request may sit out steps."""
    toks = traces.make_requests(256, [40, 30], seed=2)
    a, b = toks["r0"], toks["r1"]
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:20], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": b[:29], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": a[20:], "want": [19]}, {"id": "b", "tokens": b[29:], "want": [0]}],
         "end": ["a", "b"]},
    ]
    out_dir = str(tmp_path / "out")
    _run_trace_run(model_dirs["A"], "float32", steps, out_dir, 128)
    assert sorted(os.listdir(out_dir)) == ["2.f32"]
    cfg, w = load_plain_weights(model_dirs["A"])
    data = torch.from_numpy(np.fromfile(os.path.join(out_dir, "2.f32"), dtype="<f4").reshape(2, 256).copy())
    assert float((data[0].double() - plain_impl.forward(cfg, w, a)[-1]).abs().max()) < TOL_F32
    assert float((data[1].double() - plain_impl.forward(cfg, w, b)[-1]).abs().max()) < TOL_F32


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_padded_step_gives_the_same_bits_run_captured_and_replayed(model_dirs, tiny_configs, dtype):
    """A step of a shape that comes again is padded the same way whether it is run launch by launch (first
    sighting), run and captured (second) or replayed (third and later): the same kernels on the same shapes, so
    the logits of the same tokens are the same bits every time — and the padding's rows and requests leave no
    trace: the cache is whole afterwards and no error is reported."""
    from pih_b200.engine import StepEntry
    from pih_b200.engine.factory import create_runner
    name = "B"
    vocab = tiny_configs[name]["vocab_size"]
    toks = traces.make_requests(vocab, [50, 37, 9], seed=77)
    _, model, cache, runner = create_runner(model_dirs[name], dtype, page_size=PAGE[name], max_cache_tokens=1024,
                                            max_requests=4, cuda_graphs=True)
    assert runner.pad_steps
    outs = []
    for turn in range(4):
        rids = [f"{rid}-{turn}" for rid in toks]
        (a, ta), (b, tb), (c, tc) = [(r, t) for r, t in zip(rids, toks.values())]
        runner.step([StepEntry(a, ta[:30], []), StepEntry(c, tc[:8], [])])            # contexts for the mixed step
        # 20 + 37 + 1 rows of three requests: padded to 64 rows and four requests
        out = runner.step([StepEntry(a, ta[30:], [19]), StepEntry(b, tb, [36]), StepEntry(c, tc[8:], [0])])
        outs.append(out.float().cpu().clone())
        for r in rids:
            runner.finish(r)
    model.rt.ops.check_errors()
    cache.check()
    assert any(k[0] == "padded" and k[1] == 64 and k[2] == 4 for k in runner._graphs), list(runner._graphs)
    for later in outs[1:]:
        assert torch.equal(later, outs[0])
    assert all(f == cache.num_pages for f in cache.num_free_pages())


def test_graphs_of_padded_shapes_are_dropped_and_made_again(model_dirs, tiny_configs):
    """Only the most recently used graphs of non-decode shapes are kept; with room for two, a run over five
    shapes, each met five times in turn, drops and recaptures graphs all the time — every logit still matches the
    plain implementation, and the logits of a step are the same bits each time its shape comes round."""
    from pih_b200.engine import StepEntry
    from pih_b200.engine.factory import create_runner
    name, dtype = "A", "float32"
    vocab = tiny_configs[name]["vocab_size"]
    _, model, cache, runner = create_runner(model_dirs[name], dtype, page_size=16, max_cache_tokens=2048,
                                            max_requests=4, cuda_graphs=True)
    runner.GRAPH_LIMIT = 2
    lengths = [20, 40, 70, 140, 200]                                     # rows buckets 32, 64, 128, 192, 256
    prompts = traces.make_requests(vocab, lengths, seed=91)
    cfg, w = load_plain_weights(model_dirs[name])
    truth = {rid: plain_impl.forward(cfg, w, toks)[[len(toks) - 1]] for rid, toks in prompts.items()}
    seen = {}
    captures = 0
    for turn in range(5):
        for rid, toks in prompts.items():
            before = set(runner._graphs)
            out = runner.step([StepEntry((rid, turn), toks, [len(toks) - 1])]).float().cpu().clone()
            captures += len(set(runner._graphs) - before)
            runner.finish((rid, turn))
            compare({rid: out}, {rid: truth[rid]}, dtype, f"turn {turn} {rid}")
            assert torch.equal(out, seen.setdefault(rid, out))
            assert sum(1 for k in runner._graphs if k[0] != "decode") <= 2
    model.rt.ops.check_errors()
    cache.check()
    assert captures >= 8, captures                                        # shapes were captured more than once
