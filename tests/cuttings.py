"""Ways of cutting the same requests into steps, in the trace-replay line format.

Every function returns (steps, max_tokens): ``steps`` is a list of dicts
``{"step", "entries": [{"id", "tokens", "want"}], "end"}`` and ``max_tokens`` the
most tokens live requests hold at any time, each rounded up to 64.  In every
step all places are wanted, so each (request, position) is checked once.
"""
import random


def _round64(n):
    return -(-n // 64) * 64


def whole(seqs):
    """Each request alone, its whole sequence in one step."""
    steps = []
    for i, (rid, toks) in enumerate(seqs.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks,
                                              "want": list(range(len(toks)))}], "end": [rid]})
    return steps, max(_round64(len(t)) for t in seqs.values())


def tail_decode(seqs, tail=32):
    """Most of each request in one step, then its last ``tail`` tokens one by one."""
    steps, n = [], 0
    for rid, toks in seqs.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[:head],
                                              "want": list(range(head))}], "end": []})
        n += 1
        for j in range(head, len(toks)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [toks[j]], "want": [0]}],
                          "end": [rid] if j == len(toks) - 1 else []})
            n += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps, max(_round64(len(t)) for t in seqs.values())


def portions(seqs, sizes=(7, 2, 19, 3, 2, 31, 5, 2, 11)):
    """Each request alone, in portions of changing size, down to two tokens."""
    steps, n = [], 0
    for rid, toks in seqs.items():
        pos, k = 0, 0
        while pos < len(toks):
            c = min(sizes[k % len(sizes)], len(toks) - pos)
            k += 1
            steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[pos:pos + c],
                                                  "want": list(range(c))}],
                          "end": [rid] if pos + c == len(toks) else []})
            pos += c
            n += 1
    return steps, max(_round64(len(t)) for t in seqs.values())


def mixed(seqs, seed=0, max_live=4, decode_tail=12):
    """Up to ``max_live`` requests at a time: portions of some beside single tokens of others,
    requests sometimes sitting a step out; a finished request's place (and pages) go to the next.
    The last ``decode_tail`` tokens of every request are fed one by one."""
    rng = random.Random(seed)
    waiting = list(seqs.items())
    live = {}                       # rid -> position
    steps, n, peak = [], 0, 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, _ = waiting.pop(0)
            live[rid] = 0
        peak = max(peak, sum(_round64(len(seqs[r])) for r in live))
        entries, end = [], []
        for rid in list(live):
            toks, pos = seqs[rid], live[rid]
            if rng.random() < 0.2 and len(live) > 1:
                continue                              # sits this step out
            left = len(toks) - pos
            if left <= decode_tail:
                c = 1
            else:
                c = min(rng.choice([2, 3, 5, 8, 13, 21, 40]), left - decode_tail)
            entries.append({"id": rid, "tokens": toks[pos:pos + c], "want": list(range(c))})
            live[rid] = pos + c
            if pos + c == len(toks):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append({"step": n, "entries": entries, "end": end})
            n += 1
    return steps, peak
