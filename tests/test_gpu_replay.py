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

LENGTHS = {"A": [70, 45, 90, 33, 61, 50, 77, 40], "B": [64, 33, 97, 41, 80, 55, 35, 66]}
PAGE = {"A": 16, "B": 8}
FAMILIES = ["whole", "tail_decode", "portions", "mixed"]

# 32-bit: accumulation-order noise only (logits are O(1)).
TOL_F32 = 2e-5
# bfloat16: compared with the plain implementation rounding at the same places; two such
# implementations differ where an accumulation order flips a bf16 rounding.  Measured between
# two CPU implementations on these configurations: 1.5 % (A) and 2.8 % (B) of the logits'
# standard deviation at the worst position; the bound is 5 % at the worst position and 0.6 %
# on average.
TOL_BF16_MAX, TOL_BF16_MEAN = 0.05, 0.006

_REF = {}


def reference(model_dir, name, requests, rounding):
    key = (name, rounding)
    if key not in _REF:
        cfg, w = load_plain_weights(model_dir)
        _REF[key] = {rid: plain_impl.forward(cfg, w, toks, rounding) for rid, toks in requests.items()}
    return _REF[key]


def compare(got, ref, dtype, what):
    for rid in ref:
        g, r = got[rid].double(), ref[rid]
        assert g.shape == r.shape, (what, rid, g.shape, r.shape)
        err = (g - r).abs()
        if dtype == "float32":
            worst = int(err.max(dim=1).values.argmax())
            assert float(err.max()) < TOL_F32, f"{what} {rid}: max abs error {float(err.max()):.3e} at position {worst}"
        else:
            spread = float(r.std())
            per_pos = err.max(dim=1).values / spread
            worst = int(per_pos.argmax())
            assert float(per_pos.max()) < TOL_BF16_MAX, \
                f"{what} {rid}: error {float(per_pos.max()):.4f} of the spread at position {worst}"
            assert float(err.mean()) / spread < TOL_BF16_MEAN, f"{what} {rid}: mean error {float(err.mean()) / spread:.4f}"


@pytest.fixture(scope="module")
def requests_of(tiny_configs):
    return {n: traces.make_requests(tiny_configs[n]["vocab_size"], LENGTHS[n], seed=11) for n in ("A", "B")}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
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
    ref = reference(model_dirs[name], name, requests, "none" if dtype == "float32" else "bf16")
    compare(got, ref, dtype, f"{name} {family}")
    cache.check()
    assert all(f == cache.num_pages for f in cache.num_free_pages())
    if family == "mixed":
        assert all(g.pool.pages_handed_out > g.pool.num_pages for g in cache.groups)


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
            bound = 1e-6 if dtype == "float32" else 0.05 * float(outs["whole"][rid].std())
            assert diff <= bound, (family, rid, diff)


def _run_trace_run(model_dir, dtype, steps, out_dir, max_tokens, env=None):
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens)]
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [ln for ln in proc.stdout.splitlines() if ln.startswith("done ")] == [f"done {s['step']}" for s in steps]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(model_dirs, requests_of, tmp_path, dtype):
    """bin/trace_run with its default page size of 16, mixed trace, pool = the peak of live tokens."""
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
    ref = reference(model_dirs[name], name, requests, "none" if dtype == "float32" else "bf16")
    compare(got, ref, dtype, f"trace_run {dtype}")


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
