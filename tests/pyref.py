"""A second, independent restatement of sample_with in scalar numpy float32, used only to
cross-check the C++ oracle on small inputs (two transcriptions of
crates/llm-core/src/generate.rs:325-420 must agree). exp is the correctly rounded one
(float64 exp rounded to float32), i.e. the oracle's EXP_CR definition."""
import math

import numpy as np

F = np.float32
EOS = 258
GAMMA = 0x9E3779B97F4A7C15
M64 = (1 << 64) - 1


def next_f32(state):
    state = (state + GAMMA) & M64
    z = state
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
    z ^= z >> 31
    return state, F(z >> 40) / F(1 << 24)


def exp_cr(x):
    x = float(x)
    if math.isnan(x):
        return F(np.nan)
    try:
        return F(math.exp(x))
    except OverflowError:
        return F(np.inf)


def sample_with(logits, temperature, top_k, top_p, min_p, penalty, recent, state, allowed=None):
    """Returns (token, new_state, kept_ids, kept_probs)."""
    temperature, top_p, min_p, penalty = F(temperature), F(top_p), F(min_p), F(penalty)
    work = [F(v) for v in logits]
    n = len(work)
    if allowed is not None:
        for i in range(n):
            ok = bool(allowed[i]) if i < len(allowed) else True
            if i != EOS and not ok:
                work[i] = F(-np.inf)
    if penalty != F(1.0):
        for t in recent:
            if t < n:
                work[t] = work[t] / penalty if work[t] > F(0.0) else work[t] * penalty
    if temperature <= F(0.0):
        best, best_val = 0, F(-np.inf)
        for i, v in enumerate(work):
            if v > best_val:
                best_val, best = v, i
        return best, state, [], []
    with np.errstate(all="ignore"):
        work = [v / temperature for v in work]
    order = sorted(range(n), key=lambda i: (-float(work[i]), i))  # -0.0 and 0.0 tie as floats
    if top_k > 0:
        order = order[:top_k]
    mx = F(-np.inf)
    for i in order:
        mx = max(mx, work[i])
    with np.errstate(all="ignore"):
        probs = [exp_cr(work[i] - mx) for i in order]
    s = F(0.0)
    for p in probs:
        s = F(s + p)
    if s <= F(0.0) or not np.isfinite(s):
        return (order[0] if order else 0), state, [], []
    probs = [F(p / s) for p in probs]
    if min_p > F(0.0):
        thr = F(min_p * probs[0])
        keep = 0
        while keep < len(probs) and probs[keep] >= thr:
            keep += 1
        keep = max(keep, 1)
        probs, order = probs[:keep], order[:keep]
    if top_p < F(1.0):
        cum = F(0.0)
        keep = len(probs)
        for i, p in enumerate(probs):
            cum = F(cum + p)
            if cum >= top_p:
                keep = i + 1
                break
        probs, order = probs[:keep], order[:keep]
    total = F(0.0)
    for p in probs:
        total = F(total + p)
    state, u = next_f32(state)
    r = F(u * total)
    for i, p in enumerate(probs):
        if r < p:
            return order[i], state, order, probs
        r = F(r - p)
    return order[-1], state, order, probs
