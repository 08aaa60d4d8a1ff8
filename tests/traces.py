"""Builds replay traces (lists of steps in bin/trace_run's format) that feed the
same requests in different ways, and collects the logits they return by
(request, position)."""
import numpy as np


def whole(requests):
    """Each request alone, all of it in one step."""
    steps = []
    for rid, toks in requests.items():
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": list(toks), "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def tail_one_by_one(requests, tail=32):
    """Most of a request in one step, its last `tail` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        n = len(toks)
        head = max(n - tail, 1) if n > 1 else 1
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": list(toks[:head]), "want": list(range(head))}],
                      "end": [rid] if head == n else []})
        for i in range(head, n):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}],
                          "end": [rid] if i == n - 1 else []})
    return steps


def portions(requests, sizes=(13, 2, 7, 31, 3, 64, 5, 2, 17)):
    """Each request alone in portions of changing size, down to two tokens."""
    steps = []
    for rid, toks in requests.items():
        i, k, n = 0, 0, len(toks)
        while i < n:
            m = min(sizes[k % len(sizes)], n - i)
            k += 1
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": list(toks[i:i + m]), "want": list(range(m))}],
                          "end": [rid] if i + m == n else []})
            i += m
    return steps


def mixed(requests, prompt_frac=0.6, portion_sizes=(11, 5, 23, 2, 9), max_live=4, seed=0):
    """Up to `max_live` requests at a time: prompts fed in portions beside other
    requests' single tokens; a request now and then sits a step out; finished
    requests end so that their pages go to the ones that start later."""
    rng = np.random.default_rng(seed)
    pending = list(requests.items())
    live = {}   # rid -> [tokens, fed, prompt_len]
    steps = []
    k = 0
    while pending or live:
        while pending and len(live) < max_live:
            rid, toks = pending.pop(0)
            live[rid] = [list(toks), 0, max(1, int(len(toks) * prompt_frac))]
        entries, end = [], []
        for rid, st in list(live.items()):
            toks, fed, plen = st
            if len(live) > 1 and rng.random() < 0.15:
                continue    # sits this step out
            if fed < plen:
                m = min(portion_sizes[k % len(portion_sizes)], plen - fed)
                k += 1
            else:
                m = 1
            entries.append({"id": rid, "tokens": toks[fed:fed + m], "want": list(range(m))})
            st[1] = fed + m
            if st[1] == len(toks):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def max_live_tokens(steps, round_to=64):
    """The --max-tokens a trace needs: the most tokens live requests hold at any
    time, each request's count rounded up to a multiple of `round_to`."""
    held, peak = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return peak


def collect(steps, outputs):
    """outputs[i]: the array a step returned (or None). Returns {rid: {position: logits row}}."""
    fed, got = {}, {}
    for s, out in zip(steps, outputs):
        r = 0
        for e in s["entries"]:
            base = fed.get(e["id"], 0)
            for w in e.get("want", []):
                got.setdefault(e["id"], {})[base + w] = out[r]
                r += 1
            fed[e["id"]] = base + len(e["tokens"])
        assert out is None or r == out.shape[0]
        for rid in s["end"]:
            fed.pop(rid, None)
    return got


def as_matrix(got_for_request, n):
    assert sorted(got_for_request) == list(range(n)), "not every position was returned"
    return np.stack([got_for_request[i] for i in range(n)])
