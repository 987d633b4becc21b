"""Traces for the replay tests: the same requests cut into steps in different ways.

A trace is a list of steps ``{"step": i, "entries": [{"id", "tokens", "want"}], "end": [...]}``
— the format that ``bin/trace_run`` reads.  Every builder asks for the logits
of every token it feeds, so each family can be compared position by
position with the plain implementation's whole-sequence logits.
"""
import random

import torch


def make_requests(vocab, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(lengths)}


def whole(requests):
    """Each request alone and whole: one step, all rows wanted."""
    steps = []
    for rid, toks in requests.items():
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def tail_decode(requests, tail=32):
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        cuts = [head] + [1] * (len(toks) - head)
        pos = 0
        for i, n in enumerate(cuts):
            steps.append({"step": len(steps),
                          "entries": [{"id": rid, "tokens": toks[pos:pos + n], "want": list(range(n))}],
                          "end": [rid] if i == len(cuts) - 1 else []})
            pos += n
    return steps


def portions(requests, seed=0, sizes=(7, 2, 5, 3, 16, 2, 9, 17, 4, 2, 31)):
    """Portions of changing size, down to two tokens."""
    rnd = random.Random(seed)
    steps = []
    for rid, toks in requests.items():
        pos, k = 0, rnd.randrange(len(sizes))
        while pos < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - pos)
            k += 1
            steps.append({"step": len(steps),
                          "entries": [{"id": rid, "tokens": toks[pos:pos + n], "want": list(range(n))}],
                          "end": [rid] if pos + n == len(toks) else []})
            pos += n
    return steps


def mixed(requests, seed=0, max_live=4, decode_tail=12, max_portion=19):
    """Up to ``max_live`` requests at a time: portions of some beside single
    tokens of others; a request may sit out a step; a finished request's
    place goes to the next one, so its pages are used again."""
    rnd = random.Random(seed)
    waiting = list(requests.items())
    live = {}                       # rid -> position
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, _ = waiting.pop(0)
            live[rid] = 0
        entries, end = [], []
        for rid in list(live):
            toks = requests[rid]
            pos = live[rid]
            if len(live) > 1 and rnd.random() < 0.2:
                continue                                   # left out of this step
            remaining = len(toks) - pos
            if remaining <= decode_tail:
                n = 1
            else:
                n = min(rnd.randint(2, max_portion), remaining - decode_tail)
                if n < 2:
                    n = min(2, remaining)
            entries.append({"id": rid, "tokens": toks[pos:pos + n], "want": list(range(n))})
            live[rid] = pos + n
            if live[rid] == len(toks):
                end.append(rid)
                del live[rid]
        if not entries:
            continue
        steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def peak_tokens(steps, round_to=64):
    """Most tokens that live requests hold at any time, each rounded up to ``round_to``."""
    held, peak = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return peak


def replay(runner, steps):
    """Drive ``runner`` (a ModelRunner) through ``steps``; returns {rid: fp32 logits [len, vocab]}."""
    from pih_b200.engine import StepEntry
    rows = {}
    for s in steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]]
        logits = runner.step(entries)
        i = 0
        for e in s["entries"]:
            for _ in e["want"]:
                rows.setdefault(e["id"], []).append(logits[i].float().cpu())
                i += 1
        for rid in s["end"]:
            runner.finish(rid)
    return {rid: torch.stack(v) for rid, v in rows.items()}
