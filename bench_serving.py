#!/usr/bin/env python3
"""Continuous-batching workloads through the Python entry point, at the larger Qwen3 shapes.

    python bench_serving.py --shape 1.7b      # 32 requests, prompts of 64..2048 tokens, 256 new tokens each,
                                              # a token budget of 512 a step (prompts are cut into portions)
    python bench_serving.py --shape 8b        # 64 requests, prompts of 1024 tokens, 512 new tokens each,
                                              # greedy and temperature 0.7 mixed, untied output head

Random weights of the named architecture (seeded), seeded uniform-random prompt ids, one GPU.  Requests are all
submitted at once; the scheduler admits them, cuts their prompts under the token budget beside the decode
tokens of the others, and frees what finishes.  Prints one JSON line: generated tokens a second over the whole
run (wall clock, host in the loop; the engine's warm-up before the first request is timed apart), the same over the part of the run in which every live request decodes,
prompt tokens, steps, preemptions.  `--layers` runs fewer layers of the shape (both numbers are in the line).
"""
from __future__ import annotations

import argparse
import json
import random
import time

SHAPES = {
    "0.6b": dict(hidden_size=1024, intermediate_size=3072, num_hidden_layers=28, num_attention_heads=16,
                 num_key_value_heads=8, tie_word_embeddings=True, seed=2),
    "1.7b": dict(hidden_size=2048, intermediate_size=6144, num_hidden_layers=28, num_attention_heads=16,
                 num_key_value_heads=8, tie_word_embeddings=True, seed=3),
    "8b": dict(hidden_size=4096, intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32,
               num_key_value_heads=8, tie_word_embeddings=False, seed=4),
}
COMMON = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", torch_dtype="bfloat16", hidden_act="silu",
              use_cache=True, head_dim=128, vocab_size=151936, max_position_embeddings=40960, rope_theta=1000000.0,
              rms_norm_eps=1e-6, bos_token_id=151643, eos_token_id=151645, attention_bias=False)
WORKLOADS = {
    # requests, prompt lengths (lo, hi), new tokens, token budget a step, share of requests at temperature 0.7
    "0.6b": dict(requests=32, prompt=(64, 2048), new_tokens=256, budget=512, sampled=0.0),
    "1.7b": dict(requests=32, prompt=(64, 2048), new_tokens=256, budget=512, sampled=0.0),
    "8b": dict(requests=64, prompt=(1024, 1024), new_tokens=512, budget=4096, sampled=0.5),
}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", choices=sorted(SHAPES), default="1.7b")
    ap.add_argument("--layers", type=int, default=None, help="run this many layers of the shape")
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--requests", type=int, default=None)
    ap.add_argument("--new-tokens", type=int, default=None)
    ap.add_argument("--budget", type=int, default=None, help="tokens a step (default: the shape's workload)")
    ap.add_argument("--no-warm-up", action="store_true",
                    help="first request on a cold engine: what a process sets up and captures once falls into the run")
    ap.add_argument("--attention-in-turn", action="store_true",
                    help="a mixed step's two attention kernels one after the other instead of side by side")
    ap.add_argument("--capture-decode-after", type=int, default=None,
                    help="uncaptured runs of a decode shape before it is captured into a CUDA graph")
    args = ap.parse_args()

    import torch
    from pih_b200.config import config_from_dict
    from pih_b200.engine import Engine
    from pih_b200.kernels import get_ops
    from pih_b200.models import CausalLM, expected_tensors
    from pih_b200.parts import Runtime
    from pih_b200.sampling import SamplingParams
    from pih_b200.weights import random_tensors

    shape = dict(SHAPES[args.shape])
    seed = shape.pop("seed")
    layers_of_shape = shape["num_hidden_layers"]
    if args.layers:
        shape["num_hidden_layers"] = args.layers
    work = dict(WORKLOADS[args.shape])
    if args.requests:
        work["requests"] = args.requests
    if args.new_tokens:
        work["new_tokens"] = args.new_tokens
    if args.budget:
        work["budget"] = args.budget
    config = config_from_dict(dict(COMMON, **shape))
    spec = config.model_spec()
    dev = torch.device("cuda:0")
    rt = Runtime(dev, torch.bfloat16, get_ops(dev))
    t_build = time.perf_counter()
    model = CausalLM(spec, random_tensors(expected_tensors(spec), seed=seed, sigma=0.02, dtype=torch.bfloat16), rt)
    t_build = time.perf_counter() - t_build

    rng = random.Random(seed)
    lo, hi = work["prompt"]
    lengths = [rng.randint(lo, hi) for _ in range(work["requests"])]
    g = torch.Generator().manual_seed(seed)
    prompts = [torch.randint(0, config.vocab_size, (n,), generator=g).tolist() for n in lengths]
    # no pool size given: the engine takes what the device has left beside the weights, up to what this many
    # requests of the longest context could hold
    engine = Engine(f"Qwen3-{args.shape}-random", model=(config, model), page_size=args.page_size,
                    maximum_batch_sequences=work["requests"], maximum_batch_tokens=work["budget"],
                    maximum_context_tokens=hi + work["new_tokens"] + 32)
    if args.capture_decode_after is not None:
        engine.runner.capture_decode_after = args.capture_decode_after
    if args.attention_in_turn:
        engine.rt.ops.set_attention_side_by_side(False)
    # as a server does before it opens: the shapes that its limits make likely are run and captured once
    warm = None if args.no_warm_up else engine.warm_up()
    reqs = []
    for i, prompt in enumerate(prompts):
        sampled = i < work["sampled"] * work["requests"]
        params = SamplingParams(max_tokens=work["new_tokens"], ignore_eos=True,
                                temperature=0.7 if sampled else 0.0, seed=7 + i)
        reqs.append(engine._live[engine.submit(prompt, params)])

    import bench                                           # the clock sampler, the peaks and the weights' bytes
    torch.cuda.synchronize()
    steps = 0
    decode_only = {"steps": 0, "tokens": 0, "seconds": 0.0, "bytes": 0}
    weights = bench.weight_bytes(model)
    per_token = engine.cache.bytes_per_token()
    with bench.ClockSampler() as clocks:
        t0 = time.perf_counter()
        while engine.has_work():
            live = [r for r in reqs if r.status != "finished"]
            all_decode = all(r.num_computed >= len(r.prompt) for r in live)
            before = sum(len(r.outputs) for r in reqs)
            # what an all-decode step has to read: every weight once and the cache of the live requests
            need = weights + per_token * sum(r.num_computed for r in live)
            t = time.perf_counter()
            engine.step()
            steps += 1
            if all_decode:
                decode_only["steps"] += 1
                decode_only["tokens"] += sum(len(r.outputs) for r in reqs) - before
                decode_only["seconds"] += time.perf_counter() - t
                decode_only["bytes"] += need
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
    hbm_gbs, _, peak_source = bench.peaks()
    peaks = {"hbm_gbs": hbm_gbs, "source": peak_source}
    generated = sum(len(r.outputs) for r in reqs)
    assert all(r.status == "finished" and len(r.outputs) == work["new_tokens"] for r in reqs)
    line = {
        "metric": f"generated tok/s, continuous batching (Qwen3-{args.shape} shape)", "value": round(generated / dt, 1),
        "unit": "tok/s", "seconds": round(dt, 3), "steps": steps, "generated_tokens": generated,
        "prompt_tokens": sum(lengths), "prompt_and_generated_tok_s": round((generated + sum(lengths)) / dt, 1),
        "decode_only": {"steps": decode_only["steps"],
                        "tok_s": round(decode_only["tokens"] / decode_only["seconds"], 1) if decode_only["seconds"] else None,
                        "ms_per_step": round(decode_only["seconds"] / decode_only["steps"] * 1e3, 3) if decode_only["steps"] else None,
                        # bytes that the all-decode steps had to read / their wall time / the copy peak
                        "roofline": ({"bound": "hbm", "achieved": round(decode_only["bytes"] / decode_only["seconds"] / 1e9, 1),
                                      "peak": peaks["hbm_gbs"], "unit": "GB/s", "peaks": peaks["source"],
                                      "frac": round(decode_only["bytes"] / decode_only["seconds"] / 1e9 / peaks["hbm_gbs"], 4)}
                                     if decode_only["seconds"] else None)},
        "clocks": clocks.summary(),
        "preemptions": sum(r.preemptions for r in reqs),
        "steps_planned_ahead": engine.steps_planned_ahead, "cache_tokens": engine.cache_tokens,
        "warm_up": None if warm is None else {"seconds": warm["seconds"], "graphs": warm["graphs"]},

        "config": {"shape": args.shape, "layers": config.num_hidden_layers, "layers_of_shape": layers_of_shape,
                   "hidden": config.hidden_size, "intermediate": config.intermediate_size,
                   "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads,
                   "vocab": config.vocab_size, "tied_embeddings": config.tie_word_embeddings,
                   "requests": work["requests"], "prompt_lengths": f"{lo}..{hi}", "new_tokens": work["new_tokens"],
                   "token_budget": work["budget"], "sampled_share": work["sampled"], "dtype": "bf16",
                   "data": "synthetic", "weights_build_s": round(t_build, 1)},
        "peak_memory_gb": round(torch.cuda.max_memory_allocated() / 1e9, 2),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
