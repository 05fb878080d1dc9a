"""Ways of cutting the same requests into steps, for the replay tests.

Every function returns a list of steps; a step is (entries, end) with entries
[{"id", "tokens", "want"}].  Every position's logits are wanted, so each is compared.
"""
from __future__ import annotations

import random


def whole(requests: dict[str, list[int]]):
    """Each request alone and whole."""
    return [([{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], [rid])
            for rid, toks in requests.items()]


def tail_one_by_one(requests, tail=32, together=3):
    """Most of it in one step, the last ``tail`` tokens one by one.  ``together`` requests at a
    time: each gets most of its prompt in a step of its own, then their last tokens are decoded
    side by side, one token of each per step (the batch shrinks as the shorter tails end)."""
    steps = []
    names = list(requests)
    for g in range(0, len(names), together):
        group = names[g:g + together]
        done = {}
        for rid in group:
            toks = requests[rid]
            head = max(0, len(toks) - tail)
            done[rid] = head
            if head:
                steps.append(([{"id": rid, "tokens": toks[:head], "want": list(range(head))}], []))
        while done:
            entries, end = [], []
            for rid in list(done):
                toks, i = requests[rid], done[rid]
                entries.append({"id": rid, "tokens": [toks[i]], "want": [0]})
                done[rid] = i + 1
                if i + 1 == len(toks):
                    end.append(rid)
                    del done[rid]
            steps.append((entries, end))
    return steps


def changing_portions(requests, sizes=(48, 17, 2, 5, 2, 3, 31, 2, 64, 7)):
    """Portions of changing size, down to two tokens."""
    steps = []
    for rid, toks in requests.items():
        i, k = 0, 0
        while i < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - i)
            k += 1
            steps.append(([{"id": rid, "tokens": toks[i:i + n], "want": list(range(n))}],
                          [rid] if i + n == len(toks) else []))
            i += n
    return steps


def mixed(requests, seed=0, max_live=4, tail=12):
    """Up to ``max_live`` requests at a time: portions of some beside single tokens of others; a
    request may sit out a step.  Requests start as soon as an earlier one has ended."""
    rng = random.Random(seed)
    order = list(requests)
    live: dict[str, int] = {}
    steps = []
    while order or live:
        while order and len(live) < max_live and (not live or rng.random() < 0.6):
            live[order.pop(0)] = 0
        entries, end = [], []
        for rid in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue                      # left out of this step, goes on later
            toks, done = requests[rid], live[rid]
            left = len(toks) - done
            n = 1 if left <= tail else min(left - tail, rng.choice([2, 3, 5, 16, 17, 48]))
            entries.append({"id": rid, "tokens": toks[done:done + n], "want": list(range(n))})
            live[rid] = done + n
            if live[rid] == len(toks):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append((entries, end))
    return steps


def peak_tokens(steps, round_to=64) -> int:
    """The most tokens that live requests hold at any time, each rounded up to ``round_to``."""
    held: dict[str, int] = {}
    peak = 0
    for entries, end in steps:
        for e in entries:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in end:
            held.pop(rid, None)
    return peak
