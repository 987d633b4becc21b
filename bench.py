"""Benchmark of the pih_b200 engine: decode tokens per second of Qwen3-0.6B on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference]

A "step" is one decode step of the batch.  The default run has the layer
sizes of the Qwen3-0.6B configuration (28 layers, hidden 1024, 16/8 heads of
128, intermediate 3072, vocabulary 151 936, tied embeddings) with random
weights (N(0, 0.02), seed 2), a batch of 8 requests each holding 2 048
context tokens, page size 64.  It prints ONE JSON line:

* ``value``      decoded tokens per second, timed on the device with CUDA events around K
                 steps of the step function plus device sampling (no host transfer inside);
* ``e2e``        the same through the Python entry point (``Engine.step``): every step packs its
                 batch on the host, copies it from pinned memory, and reads the sampled tokens back;
* ``prefill``    one 2 048-token prompt in one step: tokens/s, ms, and the fraction of the bf16 peak, for the step
                 replayed from its CUDA graph (a shape seen before), and ``first_sight_ms`` for the same step at
                 the first sight of its shape, launched kernel by kernel;
* ``roofline``   bytes a decode step has to read (every weight once, the cache of the live
                 requests) / its time, against the measured HBM copy bandwidth;
* ``points``     decode tokens/s at batch 1 and 64.

Peaks come from MEASURED_PEAKS.json beside this file if it exists, else the
fallback 6.65 TB/s and 1.59 PFLOP/s.  Inputs (1.2 GB of weights plus the
cache) are larger than the 126 MB L2, so no flush is needed between steps.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_0_6B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "torch_dtype": "bfloat16",
    "hidden_act": "silu", "use_cache": True, "tie_word_embeddings": True,
    "hidden_size": 1024, "intermediate_size": 3072, "num_hidden_layers": 28,
    "num_attention_heads": 16, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 151936,
    "max_position_embeddings": 40960, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "bos_token_id": 151643, "eos_token_id": 151645, "attention_bias": False, "use_sliding_window": False,
}
CONTEXT = 2048
PREFILL_TOKENS = 2048
PAGE = 64
METRIC = "decode tok/s at batch 8 (Qwen3-0.6B, 2048-token contexts)"


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    hbm, flops, src = 6650.0, 1590.0, "fallback"
    def number(v, default):
        if isinstance(v, dict):                      # {"value": ...} or the like
            v = next((v[k] for k in ("value", "median", "mean") if k in v), None)
        try:
            v = float(v)
        except (TypeError, ValueError):
            return default
        return v if v > 0 else default

    try:
        with open(path) as f:
            p = json.load(f)
        if isinstance(p, dict):
            measured_hbm, measured_flops = number(p.get("hbm_gbs"), None), number(p.get("bf16_tflops"), None)
            if measured_hbm is not None and measured_flops is not None:
                hbm, flops, src = measured_hbm, measured_flops, "measured"
    except (OSError, ValueError):
        pass
    return hbm, flops, src


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.samples = []
        self._stop = threading.Event()
        self._proc = None
        self._thread = None
        self.index = index

    def __enter__(self):
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._thread = threading.Thread(target=self._read, daemon=True)
            self._thread.start()
        except OSError:
            self._proc = None
        return self

    def _read(self):
        for line in self._proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6 and parts[0].isdigit():
                self.samples.append(parts)
            if self._stop.is_set():
                break

    def __exit__(self, *exc):
        self._stop.set()
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        mhz = sorted(int(s[0]) for s in self.samples)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": int(self.samples[0][1]), "reasons": reasons,
                "samples": len(mhz)}


def build_model(layers: int):
    import torch
    from pih_b200.config import config_from_dict
    from pih_b200.kernels import get_ops
    from pih_b200.models import CausalLM, expected_tensors
    from pih_b200.parts import Runtime
    from pih_b200.weights import random_tensors

    raw = dict(QWEN3_0_6B, num_hidden_layers=layers)
    config = config_from_dict(raw)
    spec = config.model_spec()
    dev = torch.device("cuda:0")
    rt = Runtime(dev, torch.bfloat16, get_ops(dev))
    weights = random_tensors(expected_tensors(spec), seed=2, sigma=0.02, dtype=torch.bfloat16)
    return config, CausalLM(spec, weights, rt)


def weight_bytes(model) -> int:
    """Bytes of every weight a decode step reads once (the embedding table counts as the tied head)."""
    seen, total = set(), 0
    tensors = [model.head]
    for b in model.blocks:
        tensors += [b.mixer.w_qkv, b.mixer.w_o, b.ffn.w_gate_up, b.ffn.w_down, b.norm_in.weight,
                    b.norm_post.weight, b.mixer.q_norm, b.mixer.k_norm]
    tensors.append(model.final_norm.weight)
    for t in tensors:
        if t is not None and t.data_ptr() not in seen:
            seen.add(t.data_ptr())
            total += t.numel() * t.element_size()
    return total


def decode_run(model, batch: int, steps: int, warmup: int, context: int = CONTEXT, repeats: int = 5):
    """Device-timed decode: ``batch`` requests with ``context`` tokens in the cache
    (synthetic keys and values), one token each per step, greedy sampling on the device.  The timed loop of
    ``steps`` steps runs ``repeats`` times back to back; the median loop is reported."""
    import torch
    from pih_b200.cache import CacheManager
    from pih_b200.engine import ModelRunner, StepEntry

    spec = model.spec
    rt = model.rt
    total = steps * repeats + warmup
    cache = CacheManager(model.cache_needs(), [e.reads_cache_of for e in spec.schedule], page_size=PAGE,
                         num_pages=batch * (-(-(context + total + 1) // PAGE)), max_requests=batch,
                         device=rt.device, dtype=rt.dtype)
    for grp in cache.groups:
        grp.kv.normal_(0.0, 1.0)
    for r in range(batch):
        cache.add_request(r)
        cache.append(r, context)
        cache.commit(r)
    runner = ModelRunner(model, cache, cuda_graphs=True)
    g = torch.Generator().manual_seed(5)
    tokens = torch.randint(0, spec.vocab, (batch,), generator=g).tolist()

    def one_step(tokens):
        logits = runner.step([StepEntry(r, [tokens[r]], [0]) for r in range(batch)])
        return rt.ops.argmax(logits)

    for _ in range(warmup):
        tokens = one_step(tokens).tolist()
    loops = []
    for _ in range(repeats):
        torch.cuda.synchronize()
        launches0 = rt.ops.launches
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        # timed: the next token ids are kept as given (host list) so that no D2H sits in the region
        start.record()
        for _ in range(steps):
            out = one_step(tokens)
        stop.record()
        torch.cuda.synchronize()
        loops.append((start.elapsed_time(stop) / steps, rt.ops.launches - launches0, cache.requests[0].num_tokens))
    rt.ops.check_errors()
    ms, launches, length_after = sorted(loops)[len(loops) // 2]
    kv_bytes = batch * (length_after - steps // 2) * cache.bytes_per_token()
    del out
    for r in range(batch):
        cache.release(r)
    return {"ms": ms, "tok_s": batch / ms * 1e3, "launches": launches, "bytes": weight_bytes(model) + kv_bytes,
            "loops_ms": [round(l[0], 4) for l in loops]}


def prefill_run(model, tokens_n: int, reps: int = 6):
    import torch
    from pih_b200.cache import CacheManager
    from pih_b200.engine import ModelRunner, StepEntry

    spec, rt = model.spec, model.rt
    cache = CacheManager(model.cache_needs(), [e.reads_cache_of for e in spec.schedule], page_size=PAGE,
                         num_pages=-(-tokens_n // PAGE) + 1, max_requests=1, device=rt.device, dtype=rt.dtype)
    runner = ModelRunner(model, cache, cuda_graphs=True)    # a repeated portion shape is replayed from a graph
    g = torch.Generator().manual_seed(6)
    toks = torch.randint(0, spec.vocab, (tokens_n,), generator=g).tolist()
    # prompts of other lengths first: what the kernels and the library set up or load at their first calls with
    # rows of about this number is not part of "the first sight of a shape" in a process that has served before
    for cut in (48, 112, 16, 80):
        runner.step([StepEntry("w", toks[:tokens_n - cut], [tokens_n - cut - 1])])
        torch.cuda.synchronize()
        runner.finish("w")
    times = []
    first_sight = None
    for i in range(reps + 2):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        runner.step([StepEntry("p", toks, [tokens_n - 1])])
        stop.record()
        torch.cuda.synchronize()
        runner.finish("p")
        if i == 0:                                           # a shape not seen before: run as it is, launch by launch
            first_sight = start.elapsed_time(stop)
        if i >= 2:                                           # (the second run captures)
            times.append(start.elapsed_time(stop))
    rt.ops.check_errors()
    ms = sorted(times)[len(times) // 2]
    # flops: 2 * tokens * linear parameters + causal attention (QK^T and PV) + one row of the head
    lin = sum(t.numel() for b in model.blocks for t in (b.mixer.w_qkv, b.mixer.w_o, b.ffn.w_gate_up, b.ffn.w_down))
    a = model.blocks[0].mixer.spec
    attn = len(model.blocks) * 4 * a.heads * a.head_dim * tokens_n * (tokens_n + 1) // 2
    flops = 2 * tokens_n * lin + attn + 2 * model.head.numel()
    return {"ms": ms, "tok_s": tokens_n / ms * 1e3, "flops": flops, "first_sight_ms": first_sight}


def e2e_run(config, model_dir_weights, batch: int, steps: int, warmup: int):
    """Through the Python entry point: submit prompts, let the engine prefill, then time decode steps
    wall-clock; each step packs and copies its batch from pinned host memory and reads tokens back."""
    import torch
    from pih_b200.engine import Engine
    from pih_b200.sampling import SamplingParams

    engine = Engine(model_dir_weights, "bfloat16", page_size=PAGE, maximum_batch_sequences=batch,
                    maximum_batch_tokens=4096, maximum_context_tokens=2 * CONTEXT,    # the pool: sized by the engine
                    capture_decode_after=0)        # the batch never changes: its graph is captured at once
    g = torch.Generator().manual_seed(7)
    # long enough that no request finishes inside the timed region (prompts finish prefill on different steps)
    params = SamplingParams(max_tokens=steps + warmup + batch + 16, ignore_eos=True)
    reqs = []
    for _ in range(batch):
        rid = engine.submit(torch.randint(0, config.vocab_size, (CONTEXT,), generator=g).tolist(), params)
        reqs.append(engine._live[rid])
    while any(r.num_computed < len(r.prompt) for r in reqs):
        engine.step()
    for _ in range(warmup - 1):
        engine.step()
    torch.cuda.synchronize()
    # what the process has allocated so far (weights' tensor lists, the earlier runs' graphs) is set aside, as a
    # serving process does after start-up: a full collection over it inside the timed steps is a pause of
    # milliseconds that belongs to this script's earlier runs, not to a step
    gc.collect()
    gc.freeze()
    before = sum(len(r.outputs) for r in reqs)
    t0 = time.perf_counter()
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    gc.unfreeze()
    produced = sum(len(r.outputs) for r in reqs) - before
    assert produced == batch * steps, (produced, batch, steps)
    h2d = engine.runner.builder.last_bytes
    return {"value": produced / dt, "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * batch,
            "ms_per_step": dt / steps * 1e3}


def reference_arm():
    print(json.dumps({"impl": "reference", "unavailable":
                      "pip installs only pih_client, an HTTP client; the engine is a C++20/CUDA worker (CMake) whose "
                      "kernels are built as sm_89/sm_90 cubins only, which a B200 (sm_100) cannot load, and which "
                      "its own docs call unverified on any GPU"}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=28)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--skip-prefill", action="store_true")
    ap.add_argument("--plain-launches", action="store_true",
                    help="launch kernels fully serialised instead of with programmatic dependent launch")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    hbm_gbs, bf16_tflops, peak_src = peaks()
    config, model = build_model(args.layers)
    if args.plain_launches:
        model.rt.ops.set_dependent_launch(False)
    with ClockSampler() as clocks:
        main_run = decode_run(model, args.batch, args.steps, args.warmup)
        clock_summary = clocks.summary()
    # the end-to-end number directly after the device-timed one, with its own clock record: measured after the
    # batch-64 and prompt runs below it came out 6 % lower (1.21 against 1.15 ms a step) with nothing else changed
    e2e = None
    if not args.skip_e2e:
        from pih_b200.weights import write_random_model
        with tempfile.TemporaryDirectory() as d:
            write_random_model(d, config, seed=2, sigma=0.02)
            with ClockSampler() as clocks:
                e2e = e2e_run(config, d, args.batch, args.steps, args.warmup)
                e2e["sm_mhz"] = clocks.summary()["sm_mhz"]
        torch.cuda.empty_cache()
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = round(decode_run(model, b, max(8, args.steps // 2), 3, repeats=3)["tok_s"], 1)
    pre = None if args.skip_prefill else prefill_run(model, PREFILL_TOKENS)
    achieved = main_run["bytes"] / (main_run["ms"] * 1e-3) / 1e9
    line = {
        "metric": METRIC.replace("batch 8", f"batch {args.batch}"), "value": round(main_run["tok_s"], 1), "unit": "tok/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(main_run["ms"], 4),
        "timed_loops_ms_per_step": main_run["loops_ms"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {"model": "Qwen3-0.6B random weights seed 2", "layers": args.layers, "layers_of_config": 28,
                   "hidden": config.hidden_size, "heads": config.num_attention_heads,
                   "kv_heads": config.num_key_value_heads, "head_dim": config.head_dim,
                   "intermediate": config.intermediate_size, "vocab": config.vocab_size,
                   "tied_embeddings": config.tie_word_embeddings, "global_batch": args.batch, "seq_len": CONTEXT,
                   "context_window": 4096, "page_size": PAGE, "prefill_tokens": PREFILL_TOKENS,
                   "parallelism": "single GPU", "l2": "inputs larger than L2", "peaks": peak_src},
        "e2e": e2e,
        "gpu_launches": main_run["launches"],
        "clocks": clock_summary,
        "prefill": None if args.skip_prefill else {
            "value": round(pre["tok_s"], 1), "tokens": PREFILL_TOKENS, "ms": round(pre["ms"], 3),
            "frac": round(pre["flops"] / (pre["ms"] * 1e-3) / (bf16_tflops * 1e12), 4),
            "first_sight_ms": round(pre["first_sight_ms"], 3)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s",
                     "frac": round(achieved / hbm_gbs, 4)},
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
