"""Traces for replay tests: the same requests cut into steps in different ways.

A trace is a list of steps {"step", "entries": [{"id", "tokens", "want"}], "end"} as
bin/trace_run reads them.  Every builder asks for the logits at every position, so
any two traces of the same requests can be compared row by row, and each with the
plain implementation's whole-sequence logits.
"""
from __future__ import annotations

import random


def whole(requests: dict) -> list:
    """Each request alone and whole, one step each."""
    steps = []
    for rid, toks in requests.items():
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": list(toks), "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def tail_singly(requests: dict, tail: int = 32) -> list:
    """Most of a request in one step, its last `tail` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        cuts = [head] + [1] * (len(toks) - head)
        pos = 0
        for i, c in enumerate(cuts):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": list(toks[pos:pos + c]),
                                                           "want": list(range(c))}],
                          "end": [rid] if i == len(cuts) - 1 else []})
            pos += c
    return steps


def portions(requests: dict, sizes=(16, 7, 2, 33, 5, 2, 1, 64, 3)) -> list:
    """Each request alone, in portions of changing size, down to two tokens and one."""
    steps = []
    for k, (rid, toks) in enumerate(requests.items()):
        pos, i = 0, k   # every request starts at another place of the cycle
        while pos < len(toks):
            c = min(sizes[i % len(sizes)], len(toks) - pos)
            i += 1
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": list(toks[pos:pos + c]),
                                                           "want": list(range(c))}],
                          "end": [rid] if pos + c == len(toks) else []})
            pos += c
    return steps


def mixed(requests: dict, seed: int, max_live: int = 4, decode_tail: int = 8, max_portion: int = 24) -> list:
    """Up to `max_live` requests at a time: portions of some beside single tokens of
    others; a request is sometimes left out of a step; finished requests end at once so
    that their pages are used again by the next ones."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live = {}   # id -> [tokens, pos]
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.7):
            rid, toks = waiting.pop(0)
            live[rid] = [list(toks), 0]
        entries, end = [], []
        for rid, (toks, pos) in list(live.items()):
            if len(live) > 1 and rng.random() < 0.2:
                continue   # left out of this step
            left = len(toks) - pos
            if left <= decode_tail:
                c = 1
            else:
                c = min(left - decode_tail, rng.choice([2, 2, 3, 5, 8, 13, max_portion]))
            entries.append({"id": rid, "tokens": toks[pos:pos + c], "want": list(range(c))})
            live[rid][1] = pos + c
            if pos + c == len(toks):
                end.append(rid)
                del live[rid]
        if not entries:
            continue
        steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def peak_tokens(steps: list, round_to: int = 64) -> int:
    """The --max-tokens a trace needs: most tokens live requests hold at any time, each
    request's count rounded up to a multiple of `round_to`."""
    held, peak = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return peak


def run_in_process(runner, steps: list) -> dict:
    """Drive a ModelRunner with a trace; returns {(request id, position): logits row (CPU)}."""
    from wllm_b200.engine import StepEntry
    live, pos, rows = {}, {}, {}
    for s in steps:
        entries, keys = [], []
        for e in s["entries"]:
            rid = e["id"]
            if rid not in live:
                live[rid] = runner.cache.open(rid)
                pos[rid] = 0
            entries.append(StepEntry(live[rid], e["tokens"], e["want"]))
            keys.extend((rid, pos[rid] + w) for w in e["want"])
            pos[rid] += len(e["tokens"])
        logits = runner.step(entries).float().cpu()
        assert logits.shape[0] == len(keys)
        for k, row in zip(keys, logits):
            rows[k] = row
        for rid in s["end"]:
            runner.cache.close(live.pop(rid))
        runner.cache.check()
    return rows
