"""Checks of generated tokens against the plain implementation that allow a difference only where the
plain model itself is undecided: a greedy token must be the plain model's arg-max given the tokens before
it, or lie within the precision's bound of it; a sampled token must be the plain model's draw from the same
random number, or that number must fall within rounding of the boundary between the two tokens' intervals."""
import numpy as np
import torch

import plain_lfm2 as plain
from tolerances import K


def check_greedy(cfg, w, prompt, out, dtype, what=""):
    """Teacher-forced on the engine's own tokens, so that one near-tie does not excuse what follows it."""
    seq = list(prompt) + list(out[:-1])
    ref = plain.forward(cfg, w, seq, rows=list(range(len(prompt) - 1, len(seq)))).numpy()
    tol = 2 * K[dtype] * (1 + np.abs(ref).max())
    for j, t in enumerate(out):
        best = int(ref[j].argmax())
        assert t == best or ref[j][best] - ref[j][t] <= tol, \
            f"{what}: token {j} is {t}, the plain model's is {best} with a margin of {ref[j][best] - ref[j][t]:.3e} > {tol:.3e}"


def check_sampled(cfg, w, prompt, out, dtype, *, temperature, top_k, seed, repeat_penalty, repeat_window, what=""):
    """As tools/infer's select_next (tests/plain_lfm2.py: select_next) on the plain logits given the engine's tokens."""
    rng = plain.XorShift64(seed)
    seq = list(prompt) + list(out[:-1])
    ref = plain.forward(cfg, w, seq, rows=list(range(len(prompt) - 1, len(seq))))
    eps = 8 * K[dtype]
    toks = list(prompt)
    for j, t in enumerate(out):
        cands = plain.top_k_candidates(ref[j], top_k)
        ids = [c[0] for c in cands]
        scores = np.array([c[1] for c in cands], dtype=np.float64)
        if repeat_penalty > 1.0 and repeat_window > 0:
            tail = set(toks[-repeat_window:])
            for i, c in enumerate(ids):
                if c in tail:
                    scores[i] /= repeat_penalty
        wts = np.exp((scores - scores.max()) / temperature)
        cdf = np.cumsum(wts) / wts.sum()
        r = rng.next_f32()
        pick = int(np.searchsorted(cdf, r, side="left"))
        pick = min(pick, len(ids) - 1)
        if ids[pick] != t:
            assert t in ids, f"{what}: token {j} = {t} is not among the plain model's {len(ids)} candidates"
            i = ids.index(t)
            lo, hi = (cdf[i - 1] if i else 0.0), cdf[i]
            assert lo - eps <= r <= hi + eps, \
                f"{what}: token {j} is {t} (interval {lo:.6f}..{hi:.6f}), the draw {r:.6f} gives {ids[pick]}"
        toks.append(t)
