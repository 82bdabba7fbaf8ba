"""Builders of replay traces (lists of steps in bin/trace_run's input format) and a
checker that compares what a replay wrote with the plain implementation's whole-sequence
logits, position by position."""
import random

import numpy as np


def round_up(x, m):
    return (x + m - 1) // m * m


def whole(requests):
    """Each request alone and whole, one after the other; every position wanted."""
    steps = []
    for name, toks in requests.items():
        steps.append({"step": len(steps), "entries": [{"id": name, "tokens": list(toks), "want": list(range(len(toks)))}],
                      "end": [name]})
    return steps


def tail_one_by_one(requests, tail=32):
    """Most of a request in one step, its last `tail` tokens one by one."""
    steps = []
    for name, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": len(steps), "entries": [{"id": name, "tokens": list(toks[:head]), "want": [head - 1]}], "end": []})
        for i in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": name, "tokens": [toks[i]], "want": [0]}],
                          "end": [name] if i == len(toks) - 1 else []})
        if head == len(toks):
            steps[-1]["end"] = [name]
    return steps


def portions(requests, sizes=(7, 2, 13, 3, 2, 5, 1, 9, 2, 4)):
    """Portions of changing size, down to two tokens (and single tokens)."""
    steps = []
    k = 0
    for name, toks in requests.items():
        at = 0
        while at < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - at)
            k += 1
            steps.append({"step": len(steps), "entries": [{"id": name, "tokens": list(toks[at:at + n]), "want": list(range(n))}],
                          "end": [name] if at + n == len(toks) else []})
            at += n
    return steps


def mixed(requests, seed=0, max_live=4, tail=32, max_portion=17):
    """Up to max_live requests live at once: portions of some beside single tokens of
    others, requests left out of some steps, new ones entering as others end."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live = {}           # name -> (tokens, at)
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.6):
            name, toks = waiting.pop(0)
            live[name] = [list(toks), 0]
        entries, end = [], []
        for name in list(live):
            toks, at = live[name]
            if len(live) > 1 and rng.random() < 0.25:
                continue                                    # left out of this step
            remaining = len(toks) - at
            n = 1 if remaining <= tail else min(rng.randint(2, max_portion), remaining - tail)
            entries.append({"id": name, "tokens": toks[at:at + n], "want": list(range(n))})
            live[name][1] = at + n
            if at + n == len(toks):
                end.append(name)
                del live[name]
        if not entries:
            continue
        steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def max_live_tokens(steps, quantum=64):
    """The most tokens live requests hold at any time, each rounded up to the quantum."""
    held, worst = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(round_up(n, quantum) for n in held.values()))
        for name in s["end"]:
            held.pop(name, None)
    return worst


def expected(steps, plain_logits):
    """step -> [wanted, vocab] array the replay should produce, from whole-sequence logits."""
    at, out = {}, {}
    for s in steps:
        rows = []
        for e in s["entries"]:
            start = at.get(e["id"], 0)
            for w in e["want"]:
                rows.append(plain_logits[e["id"]][start + w])
            at[e["id"]] = start + len(e["tokens"])
        for name in s["end"]:
            at.pop(name, None)
        if rows:
            out[s["step"]] = np.stack(rows)
    return out


def first_mismatch(steps, got, want, atol):
    """(step, entry id, position, error) of the first wanted place beyond atol, or None."""
    at = {}
    for s in steps:
        r = 0
        for e in s["entries"]:
            start = at.get(e["id"], 0)
            for w in e["want"]:
                err = float(np.abs(got[s["step"]][r] - want[s["step"]][r]).max())
                if not err <= atol:
                    return s["step"], e["id"], start + w, err
                r += 1
            at[e["id"]] = start + len(e["tokens"])
        for name in s["end"]:
            at.pop(name, None)
    return None
