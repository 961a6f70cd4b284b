"""Inputs chosen to push the exact-selection path through its less common branches, each against
the oracle (bit-exact bar): rows whose order defeats the running bound (ascending, so every vector
is flagged and the candidate buffer compacts round after round), rows of ties (the bound never
separates anything; the index order decides), every rank-cut class (1 value per lane up to 8 per
lane), long histories whose penalised ids outnumber the rank cut, masks that leave fewer values
than the rank cut inside a shard, and bf16 rows (shorter rounds)."""
import numpy as np
import pytest

import oracle
import parity
from scriptonait_b200.workloads import Workload, narrow_bf16

pytestmark = pytest.mark.gpu


def _wl(logits, **kw):
    B = logits.shape[0]
    kw.setdefault("seeds", np.arange(B, dtype=np.uint64) + np.uint64(4242))
    return Workload("paths", logits, batch=B, **kw)


def _check(sampler, w, kept_capacity=64, allowed=None, **kw):
    gpu = parity.run_gpu(sampler, w, kept_capacity=kept_capacity, allowed=allowed, **kw)
    rep = parity.compare(parity.run_oracle(w, oracle.EXP_CR, kept_capacity, allowed=allowed), gpu, w, exact=True)
    parity.assert_exact(rep)
    return gpu


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("top_k", [1, 40, 256, 300, 1000, 2048])
def test_ascending_rows_flag_everything(sampler, top_k, bf16):
    V = 20000
    base = np.linspace(-8.0, 8.0, V, dtype=np.float32)
    x = np.stack([base, base[::-1].copy(), np.roll(base, 7777)])
    if bf16:
        x = narrow_bf16(x)   # many ties after narrowing: value desc, index asc must still hold
    _check(sampler, _wl(x, temperature=0.9, top_k=top_k, top_p=0.97), kept_capacity=128)


@pytest.mark.parametrize("top_k", [1, 50, 257, 2048])
def test_rows_of_ties(sampler, top_k):
    V = 9000
    x = np.zeros((3, V), np.float32)
    x[1, :] = 1.5
    x[1, 100::7] = 2.5          # 1272 equal leaders, more than most rank cuts
    x[2, :] = -np.inf
    x[2, 5000:5010] = 0.25
    _check(sampler, _wl(x, temperature=1.0, top_k=top_k, top_p=0.9), kept_capacity=128)


@pytest.mark.parametrize("top_k,hist_len", [(8, 1024), (64, 1024), (500, 700), (1500, 1024)])
def test_long_histories_against_every_rank_cut_class(sampler, top_k, hist_len):
    g = np.random.default_rng(top_k)
    V = 30011
    x = g.normal(0.0, 1.5, (6, V)).astype(np.float32)
    hist = g.integers(0, V, size=(6, hist_len), dtype=np.uint32)
    hist[0, :] = hist[0, 0]                                   # one id, hist_len occurrences (compounding)
    hist[1, : hist_len // 2] = np.argsort(-x[1])[: hist_len // 2]   # the leaders are the penalised ids
    _check(sampler, _wl(x, temperature=0.8, top_k=top_k, top_p=0.95, repetition_penalty=1.3, history=hist),
           kept_capacity=128)


@pytest.mark.parametrize("split", [1, 3])
def test_mask_leaves_fewer_values_than_the_rank_cut(sampler, split):
    g = np.random.default_rng(9)
    V = 40000
    x = g.normal(0.0, 1.0, (4, V)).astype(np.float32)
    allowed = np.zeros(V, bool)
    allowed[g.choice(V, 30, replace=False)] = True            # 30 allowed ids, rank cut 64
    allowed[:8] = True
    hist = g.integers(0, V, size=(4, 64), dtype=np.uint32)
    _check(sampler, _wl(x, temperature=1.0, top_k=64, top_p=0.99, repetition_penalty=1.2, history=hist),
           allowed=allowed, split=split)


def test_bf16_rows_with_penalty_and_small_rank_cut(sampler):
    g = np.random.default_rng(12)
    V = 128256
    x = narrow_bf16(g.normal(0.0, 2.0, (5, V)).astype(np.float32))
    hist = g.integers(0, V, size=(5, 300), dtype=np.uint32)
    _check(sampler, _wl(x, temperature=0.7, top_k=50, top_p=0.9, min_p=0.02, repetition_penalty=1.15, history=hist))


def _quotient_tie(T):
    """A float x_k in [1, 2) whose lower neighbour rounds to the same quotient x / T (generate.rs:357-359)."""
    T = np.float32(T)
    for start in np.linspace(1.0, 2.0, 64, endpoint=False, dtype=np.float32):
        x = np.float32(start)
        for _ in range(64):
            below = np.nextafter(x, np.float32(-np.inf))
            if np.float32(x / T) == np.float32(below / T):
                return x, below
            x = np.nextafter(x, np.float32(np.inf))
    raise AssertionError("no pair of neighbouring floats with equal quotient found")


@pytest.mark.parametrize("T", [1.5, 0.7])
@pytest.mark.parametrize("top_k,V", [(256, 1024), (8, 32), (64, 256)])
def test_quotient_tie_below_a_tight_bound_keeps_the_lower_index(sampler, T, top_k, V):
    """The rank cut works on x / T, ties go to the lower index (generate.rs:364-370). The row
    makes the running bound tight: exactly top_k large values, one per 16-byte vector, the
    smallest of them (x_k) at a high index. A value one float below x_k with the same
    quotient sits at a lower index: the reference's top_k contains it and drops x_k."""
    x_k, below = _quotient_tie(T)
    rows = []
    for variant in range(3):
        g = np.random.default_rng(100 + variant)
        x = np.full(V, -30.0, np.float32) + g.normal(0, 0.01, V).astype(np.float32)
        slots = np.arange(top_k) * 4 + g.integers(0, 4, top_k)       # one large value per vector of four
        large = (np.float32(2.0) + g.random(top_k).astype(np.float32)).astype(np.float32)
        x[slots] = large
        x[slots[-1]] = x_k                                           # the k-th value, at a high index
        low = slots[variant] + (1 if slots[variant] % 4 != 3 else -1)  # a small slot inside an early vector
        x[low] = below
        rows.append(x)
    x = np.stack(rows)
    w = _wl(x, temperature=T, top_k=top_k, top_p=1.0)
    ref = parity.run_oracle(w, oracle.EXP_CR, kept_capacity=top_k)
    for r in range(3):  # the construction does what it says: the lower-index twin is kept, x_k is not
        kept = set(ref.kept_ids[r, :ref.kept_count[r]].tolist())
        assert int(np.flatnonzero(x[r] == below)[0]) in kept and int(np.flatnonzero(x[r] == x_k)[0]) not in kept
    _check(sampler, w, kept_capacity=top_k)
