"""Builders of replay traces: the same requests cut into steps in different ways.

A trace is a list of steps ``{"step", "entries": [{"id", "tokens", "want"}], "end"}``.
Every token's logits are wanted, so each cutting can be compared place by place with the
plain implementation run on the whole request.
"""
from __future__ import annotations

import random


def _entry(rid, tokens, lo, hi):
    return {"id": rid, "tokens": tokens[lo:hi], "want": list(range(hi - lo))}


def whole(requests: dict) -> list[dict]:
    """Each request alone and whole."""
    return [{"step": i, "entries": [_entry(r, t, 0, len(t))], "end": [r]}
            for i, (r, t) in enumerate(requests.items())]


def tail_decoded(requests: dict, tail: int = 32) -> list[dict]:
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for r, t in requests.items():
        head = max(1, len(t) - tail)
        cuts = [0, head] + list(range(head + 1, len(t) + 1))
        for lo, hi in zip(cuts, cuts[1:]):
            steps.append({"step": len(steps), "entries": [_entry(r, t, lo, hi)],
                          "end": [r] if hi == len(t) else []})
    return steps


def portions(requests: dict, sizes=(7, 2, 13, 3, 2, 29, 5, 2, 17)) -> list[dict]:
    """Portions of changing size, down to two tokens."""
    steps = []
    for r, t in requests.items():
        lo, i = 0, 0
        while lo < len(t):
            hi = min(len(t), lo + sizes[i % len(sizes)])
            steps.append({"step": len(steps), "entries": [_entry(r, t, lo, hi)],
                          "end": [r] if hi == len(t) else []})
            lo, i = hi, i + 1
    return steps


def mixed(requests: dict, seed: int = 0, max_live: int = 4) -> list[dict]:
    """Up to ``max_live`` requests at a time: portions of some beside single tokens of
    others, some left out of a step; finished requests make room for the next ones."""
    rng = random.Random(seed)
    waiting = list(requests)
    live: dict = {}
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            live[waiting.pop(0)] = 0
        entries, end = [], []
        for r in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue                                  # left out of this step
            t, lo = requests[r], live[r]
            kind = rng.random()
            n = 1 if kind < 0.45 else 2 if kind < 0.6 else rng.randint(3, 24)
            hi = min(len(t), lo + n)
            entries.append(_entry(r, t, lo, hi))
            live[r] = hi
            if hi == len(t):
                end.append(r)
                del live[r]
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def max_live_tokens(steps: list[dict], round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held: dict = {}
    worst = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(-(-n // round_to) * round_to for n in held.values()))
        for r in s["end"]:
            del held[r]
    return worst


def collect(steps: list[dict], outputs: dict) -> dict:
    """Put per-step logits ``outputs[step]`` ([wanted, vocab]) back in request order:
    returns request id -> list of (position, logits row)."""
    pos: dict = {}
    rows: dict = {}
    for s in steps:
        k = 0
        for e in s["entries"]:
            start = pos.get(e["id"], 0)
            for w in e["want"]:
                rows.setdefault(e["id"], []).append((start + w, outputs[s["step"]][k]))
                k += 1
            pos[e["id"]] = start + len(e["tokens"])
    return rows
