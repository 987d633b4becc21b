"""Trace replay: feed given token ids through the model step by step and write logits.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps come on standard input, one JSON object a line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step are one batch for the step function; ``want`` lists the
places among an entry's tokens whose logits are written; ``end`` lists the
requests that are finished after the step, whose pages go back to the pool.
For a step that wants something, ``<out>/<step>.f32`` holds the logits as
little-endian float32 ``[wanted, vocab]`` in the order of the entries and of
``want``.  After every step ``done <step>`` is printed and flushed.

Nothing is sampled.  The program has no forward pass, cache or loader of its
own: it drives ``pih_b200.engine.factory.create_runner`` — the model, step
function, cache manager and kernels that generation uses.  The reference has
no such program; its nearest relatives are ``--generate-tokens``
(src/worker/main.cpp:40-77, final ids only) and the tap suite
(plugins/model-qwen3/qwen3_bf16_tap_suite_plan.cpp:17-71, hashes of fixed
positions).
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    from ..cache import DEFAULT_PAGE_SIZE
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--page-size", type=int, default=DEFAULT_PAGE_SIZE)
    ap.add_argument("--max-requests", type=int, default=64)
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    if args.max_tokens < 1:
        ap.error("--max-tokens must be >= 1")

    import torch
    from ..engine.batch import StepEntry
    from ..engine.factory import create_runner

    os.makedirs(args.out, exist_ok=True)
    _, model, cache, runner = create_runner(
        args.model, args.dtype, device=args.device, page_size=args.page_size,
        max_cache_tokens=args.max_tokens, max_requests=args.max_requests)
    ops = model.rt.ops
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", [])) for e in rec.get("entries", [])]
        if entries:
            logits = runner.step(entries)
            if logits is not None:
                host = logits.to(torch.float32).cpu().numpy()
                ops.check_errors()
                host.astype("<f4", copy=False).tofile(os.path.join(args.out, f"{step}.f32"))
            else:
                torch.cuda.synchronize()
                ops.check_errors()
        for rid in rec.get("end", []):
            runner.finish(rid)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
