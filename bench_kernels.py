"""Times single kernels of the pack at the benchmark's sizes (Qwen3-0.6B shapes by default).

    python bench_kernels.py attn_decode --batch 8 --ctx 2048
    python bench_kernels.py attn_prefill --tokens 2048
    python bench_kernels.py linear --m 8 --n 4096 --k 1024
    python bench_kernels.py rmsnorm|qk|silu --rows 8

Each kernel is timed with CUDA events on the launching stream after warm-up;
between timed launches a buffer larger than the 126 MB L2 is written so that
inputs come from HBM.  Prints one JSON line with the time, the algorithmic
bytes or flops and the achieved rate.  It is the small case that the ncu
summaries under profiles/ were captured on.  Event times of one launch come in
steps of a few microseconds on this hardware; for kernels of that size use
``--chain``: many calls on different inputs (together larger than L2) back to back in
one CUDA graph, which gives the time of one call as a step sees it.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
from types import SimpleNamespace

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def time_kernel(fn, iters, flush=True):
    import torch
    junk = torch.empty(160 * 1024 * 1024, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if junk is not None:
            junk.fill_(1)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        stop.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(stop) * 1e3)
    times.sort()
    return times[len(times) // 2]


def step_of(lens, new, dev):
    import torch
    cu = [0]
    for n in new:
        cu.append(cu[-1] + n)
    starts = [l - n for l, n in zip(lens, new)]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    return SimpleNamespace(num_requests=len(lens), cu_q=i32(cu), q_start=i32(starts), host_cu_q=cu,
                           host_q_start=starts, attention_plans={}, meta=i32([max(lens), sum(new), len(lens), 0]),
                           request_of_row=i32([r for r, n in enumerate(new) for _ in range(n)]),
                           positions=i32([starts[r] + i for r, n in enumerate(new) for i in range(n)]))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["attn_decode", "attn_prefill", "linear", "rmsnorm", "qk", "silu", "argmax", "sample"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--ctx-min", type=int, default=0, help="attn_decode: the shortest context (default: all --ctx)")
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--start", type=int, default=0, help="attn_prefill: tokens of the request already in the cache")
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page", type=int, default=64)
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=1024)
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--top-p", type=float, default=1.0, help="sample: nucleus share")
    ap.add_argument("--top-k", type=int, default=0, help="sample: keep this many (0: all)")
    ap.add_argument("--width", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--impl", default="default", choices=["default", "tcgen05", "tcgen05pair", "skinny", "library"])
    ap.add_argument("--fused", default="none", choices=["none", "norm", "addnorm", "swiglu", "residual"],
                    help="linear --impl skinny: with the RMSNorm prologue (addnorm: and the residual add before it; "
                         "swiglu: and the SwiGLU epilogue), or with the residual add in the epilogue")
    ap.add_argument("--tile-n", type=int, default=0)
    ap.add_argument("--out-f32", action="store_true", help="linear: 32-bit output, as the output head has")
    ap.add_argument("--chain", action="store_true", help="many calls on different inputs back to back in a CUDA graph: the time of one call inside a step")
    ap.add_argument("--chain-mb", type=float, default=200.0,
                    help="--chain: total size of the distinct weights (below the L2 size they stay resident)")
    ap.add_argument("--split", type=int, default=0, help="keys per split of the decode attention (0: automatic)")
    ap.add_argument("--no-tma", action="store_true", help="decode attention gathers with cp.async instead of TMA")
    ap.add_argument("--tickets", action="store_true",
                    help="decode attention merges its splits through scratch memory and tickets, not as a cluster")
    ap.add_argument("--fetched-merge", action="store_true",
                    help="decode attention: the cluster's blocks fetch one another's partials even where they would send them")
    ap.add_argument("--plain", action="store_true", help="the pack's plain (generic / FMA) kernel instead")
    args = ap.parse_args()

    import torch
    from pih_b200.kernels import get_ops
    dev = torch.device("cuda:0")
    ops = get_ops(dev)
    bf = torch.bfloat16
    H, KV, D, P = args.heads, args.kv_heads, args.head_dim, args.page
    ops.attention_split = args.split
    ops.tma_attention = not args.no_tma
    if args.impl == "skinny":
        ops.set_skinny_rule(False)                    # the kernel itself, also where the engine would not use it
    if args.tickets:
        ops.set_attention_cluster_merge(False)
    elif args.fetched_merge:
        ops.set_attention_cluster_merge("fetched")
    out = {"kernel": args.kernel}

    scale = 1.0 / math.sqrt(D)
    rates = {}                                        # filled by make(): algorithmic bytes / flops of one call

    def make():
        """One call of the chosen kernel on inputs of its own; returns (closure, bytes the inputs occupy)."""
        k = args.kernel
        if k in ("attn_decode", "attn_prefill"):
            if k == "attn_decode":
                lo = args.ctx_min or args.ctx                       # contexts spread evenly from --ctx-min to --ctx
                lens = [lo + (args.ctx - lo) * i // max(1, args.batch - 1) for i in range(args.batch)]
                new = [1] * args.batch
            else:
                lens, new = [args.start + args.tokens], [args.tokens]      # a portion that starts at --start
            pages_per = [-(-n // P) for n in lens]
            num_pages = sum(pages_per)
            cache = torch.randn(num_pages, 2, KV, P, D, device=dev).to(bf)
            table = torch.full((len(lens), max(pages_per)), -1, dtype=torch.int32)
            perm = torch.randperm(num_pages).tolist()
            for r, n in enumerate(pages_per):
                table[r, :n] = torch.tensor([perm.pop() for _ in range(n)], dtype=torch.int32)
            table = table.to(dev)
            q = torch.randn(sum(new), (H + 2 * KV) * D, device=dev).to(bf)
            step = step_of(lens, new, dev)
            if k == "attn_decode":
                rates.update(bytes=sum(lens) * 2 * KV * D * 2, batch=args.batch, ctx=args.ctx)
            else:
                rates.update(flops=4 * H * D * (args.tokens * (args.tokens + 1) // 2 + args.tokens * args.start),
                             tokens=args.tokens, start=args.start)
            if args.plain:
                fn = lambda: ops.paged_attention_generic(q, heads=H, kv_heads=KV, head_dim=D, kv_cache=cache,
                                                         block_table=table, request_of_row=step.request_of_row,
                                                         positions=step.positions, scale=scale, window=0)
            else:
                fn = lambda: ops.paged_attention_mma(q, heads=H, kv_heads=KV, head_dim=D, kv_cache=cache,
                                                     block_table=table, step=step, scale=scale, window=0)
            return fn, cache.numel() * 2
        if k == "linear":
            x = torch.randn(args.m, args.k, device=dev).to(bf)
            w = torch.randn(args.n, args.k, device=dev).to(bf)
            rates.update(flops=2 * args.m * args.n * args.k, m=args.m, n=args.n, k=args.k,
                         bytes=2 * (args.m * args.k + args.n * args.k + args.m * args.n))
            if args.impl in ("tcgen05", "tcgen05pair") and args.fused == "swiglu":
                fn = lambda: ops.linear_tcgen05_swiglu(x, w)             # (on pairs of SMs whichever of the two is named)
            elif args.impl == "library" and args.fused == "swiglu":
                fn = lambda: ops.silu_mul(torch.mm(x, w.t()), 8)
            elif args.impl in ("tcgen05", "tcgen05pair"):
                fn = lambda: ops.linear_tcgen05(x, w, tile_n=args.tile_n, pairs=args.impl == "tcgen05pair")
            elif args.impl == "skinny" and args.fused == "residual":
                r = torch.randn(args.m, args.n, device=dev).to(bf)
                fn = lambda: ops.linear_skinny(x, w, residual=r)
            elif args.impl == "skinny" and args.fused != "none":
                d = torch.randn(args.m, args.k, device=dev).to(bf) if args.fused == "addnorm" else None
                nw = torch.ones(args.k, device=dev).to(bf)
                fn = lambda: ops.linear_skinny(x, w, delta=d, norm_weight=nw, eps=1e-6, swiglu=args.fused == "swiglu")
            elif args.impl == "skinny":
                fn = lambda: ops.linear_skinny(x, w)
            elif args.impl == "library" and args.out_f32:
                rates["bytes"] += 2 * args.m * args.n
                fn = lambda: torch.mm(x, w.t(), out_dtype=torch.float32)
            elif args.impl == "library":
                fn = lambda: torch.mm(x, w.t())
            elif args.out_f32:
                rates["bytes"] += 2 * args.m * args.n
                fn = lambda: ops.linear(x, w, out_dtype=torch.float32)
            else:
                fn = (lambda: ops.linear_plain(x, w)) if args.plain else (lambda: ops.linear(x, w))
            return fn, (x.numel() + w.numel()) * 2
        if k == "rmsnorm":
            x = torch.randn(args.rows, args.width, device=dev).to(bf)
            d = torch.randn(args.rows, args.width, device=dev).to(bf)
            w = torch.ones(args.width, device=dev).to(bf)
            rates.update(bytes=args.rows * args.width * 2 * 4, rows=args.rows, width=args.width)
            return (lambda: ops.rmsnorm(x, w, 1e-6, delta=d)), x.numel() * 4
        if k == "qk":
            rows = args.rows
            qkv = torch.randn(rows, (H + 2 * KV) * D, device=dev).to(bf)
            qw = torch.ones(D, device=dev).to(bf)
            cache = torch.zeros(-(-rows // P) + 1, 2, KV, P, D, device=dev, dtype=bf)
            table = torch.zeros(4096, D // 2, 2, device=dev)
            pos = torch.arange(rows, dtype=torch.int32, device=dev) % 4096
            slots = torch.arange(rows, dtype=torch.int32, device=dev)
            rates.update(bytes=rows * ((H + 2 * KV) * D * 2 + (H + KV) * D * 2 + 2 * KV * D * 2), rows=rows)
            fn = lambda: ops.qk_norm_rope_kv_write(qkv, heads=H, kv_heads=KV, head_dim=D, q_norm=qw, k_norm=qw,
                                                   eps=1e-6, rope_table=table, rotary_dim=D, positions=pos,
                                                   slot_mapping=slots, kv_cache=cache, write_kv=True)
            return fn, (qkv.numel() + cache.numel()) * 2
        if k == "silu":
            gu = torch.randn(args.rows, 2 * 3072, device=dev).to(bf)
            rates.update(bytes=args.rows * 3072 * 2 * 3, rows=args.rows)
            return (lambda: ops.silu_mul(gu)), gu.numel() * 3
        lg = torch.randn(args.rows, 151936, device=dev) * 3.0
        rates.update(bytes=args.rows * 151936 * 4, rows=args.rows)
        if k == "sample":                               # temperature 0.7 over the whole vocabulary, top_p / top_k as given
            # the kernel alone: its per-row parameters are on the device already (temperature, top_p | top_k, seed,
            # ordinal, no suppressed ids), as pih_b200/sampling/sampler.py lays them out
            fparams = torch.tensor([[0.7, args.top_p]] * args.rows, dtype=torch.float32, device=dev)
            iparams = torch.full((args.rows, 23), -1, dtype=torch.int32)
            for i in range(args.rows):
                iparams[i, :6] = torch.tensor([args.top_k, i, 0, i, 0, 0], dtype=torch.int32)
            iparams = iparams.to(dev)
            rates.update(top_p=args.top_p, top_k=args.top_k)
            return (lambda: ops.sample(lg, fparams, iparams)), lg.numel() * 4
        return (lambda: ops.argmax(lg)), lg.numel() * 4

    if args.chain:
        # many calls on different inputs (together larger than L2 unless --chain-mb says otherwise) back to back
        # in one CUDA graph: the time of one call as a step sees it, boundaries between kernels included
        fn, size = make()
        reps = max(4, min(256, int(args.chain_mb * 1e6 / max(size, 1)) + 1))
        fns = [fn] + [make()[0] for _ in range(reps - 1)]
        for f in fns[:2]:
            f()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for f in fns:
                f()
        g.replay()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(5):
            g.replay()
        stop.record()
        torch.cuda.synchronize()
        us = start.elapsed_time(stop) * 1e3 / (5 * reps)
        out["chained"] = reps
    else:
        us = time_kernel(make()[0], args.iters, not args.no_flush)
    out["us"] = round(us, 2)
    if "flops" in rates:
        out["tflops"] = round(rates.pop("flops") / us / 1e6, 2)
    if "bytes" in rates:
        out["gbs"] = round(rates.pop("bytes") / us / 1e3, 1)
    out.update(rates)
    ops.check_errors()
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
