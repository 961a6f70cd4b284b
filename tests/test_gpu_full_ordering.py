"""The full ordering (stable radix sort + warp chains) against the oracle, bit-exact: vocabularies
that are not a multiple of the sort's tile, many equal values (the stable sort must keep ascending
indices), -inf entries, a mask and a penalty inside the full ordering, bf16 rows, top-p and min-p
cuts deep inside a flat row, and the greedy case."""
import numpy as np
import pytest

import oracle
import parity
from scriptonait_b200 import native as N
from scriptonait_b200.workloads import Workload, narrow_bf16

pytestmark = pytest.mark.gpu


def _wl(logits, **kw):
    B = logits.shape[0]
    kw.setdefault("seeds", np.arange(B, dtype=np.uint64) + np.uint64(991))
    return Workload("full", logits, batch=B, **kw)


def _check(sampler, w, allowed=None, **kw):
    gpu = parity.run_gpu(sampler, w, kept_capacity=64, allowed=allowed, **kw)
    orc = parity.run_oracle(w, oracle.EXP_CR, 64, allowed=allowed)
    assert all(f & N.ROW_FULL_SORT for f in gpu.flags), "these rows are meant to take the full ordering"
    assert np.array_equal(gpu.tokens, orc.tokens)
    assert np.array_equal(gpu.kept_count, orc.kept_count)
    assert np.array_equal(gpu.stats, orc.stats)
    return gpu


@pytest.mark.parametrize("vocab", [5001, 50257, 128256])
def test_flat_rows_of_several_sizes(sampler, vocab):
    g = np.random.default_rng(vocab)
    x = g.normal(0.0, 0.3, (3, vocab)).astype(np.float32)
    _check(sampler, _wl(x, temperature=1.0, top_k=0, top_p=0.9))
    _check(sampler, _wl(x, temperature=1.3, top_k=0, top_p=1.0, min_p=0.2))


def test_many_equal_values_keep_ascending_indices(sampler):
    g = np.random.default_rng(3)
    V = 30000
    x = g.integers(0, 7, (3, V)).astype(np.float32) * np.float32(0.25)   # seven distinct values
    x[2, ::3] = -np.inf
    _check(sampler, _wl(x, temperature=1.0, top_k=0, top_p=0.5))
    _check(sampler, _wl(narrow_bf16(x), temperature=0.7, top_k=0, top_p=0.8))


def test_mask_and_penalty_inside_the_full_ordering(sampler):
    g = np.random.default_rng(4)
    V = 20011
    x = g.normal(0.0, 0.2, (4, V)).astype(np.float32)
    hist = g.integers(0, V, size=(4, 200), dtype=np.uint32)
    hist[1, :50] = hist[1, 0]
    allowed = g.random(V) < 0.7
    w = _wl(x, temperature=0.9, top_k=0, top_p=0.95, repetition_penalty=1.4, history=hist)
    _check(sampler, w, allowed=allowed)


def test_forced_full_ordering_for_rank_cut_and_greedy_rows(sampler):
    g = np.random.default_rng(5)
    V = 9973
    x = g.normal(0.0, 2.0, (5, V)).astype(np.float32)
    hist = g.integers(0, V, size=(5, 64), dtype=np.uint32)
    _check(sampler, _wl(x, temperature=0.8, top_k=300, top_p=0.9, repetition_penalty=1.2, history=hist), force_full_sort=True)
    gpu = _check(sampler, _wl(x, temperature=0.0), force_full_sort=True)
    assert list(gpu.tokens) == list(np.argmax(x, axis=1))


@pytest.mark.parametrize("vocab", [50257, 128256])
def test_windows_too_large_for_shared_memory_but_far_from_the_whole_row(sampler, vocab):
    """Rows whose significance window holds thousands of values, not all of them: ordered from the
    window alone where that decides the row, from the whole row where it cannot (an open tail the
    draw walks into, a min-p threshold below 2^-24 of the leader)."""
    g = np.random.default_rng(vocab + 1)
    x = g.normal(0.0, 4.0, (6, vocab)).astype(np.float32)
    x[:, 7] = x.max(axis=1) + np.float32(4.0)   # a leader well above the bulk: the window ends inside the bulk's upper tail
    wide = x.astype(np.float64)
    inside = ((wide - wide.max(axis=1, keepdims=True)) >= -17.4).sum(axis=1)
    assert (inside > 4096).all() and (inside < vocab // 3).all(), inside
    _check(sampler, _wl(x, temperature=1.0, top_k=0, top_p=0.9))
    _check(sampler, _wl(x, temperature=1.0, top_k=0, top_p=1.0))                 # open tail
    _check(sampler, _wl(x, temperature=1.0, top_k=0, top_p=0.999, min_p=1e-9))   # threshold below 2^-24
    _check(sampler, _wl(x, temperature=1.0, top_k=0, top_p=1.0, min_p=0.001))
    _check(sampler, _wl(x, temperature=1.0, top_k=vocab - 5, top_p=0.95))        # a rank cut beyond exact selection
    hist = g.integers(0, vocab, size=(6, 100), dtype=np.uint32)
    _check(sampler, _wl(narrow_bf16(x), temperature=1.1, top_k=0, top_p=0.9, repetition_penalty=1.2, history=hist))


def test_more_rows_than_scratch_slots_queue_for_them(sampler):
    """One scratch slot per SM: with more undecided rows than that in a launch, CTAs wait for a slot
    (bounded polling) and every row is still resolved."""
    g = np.random.default_rng(17)
    B, V = 400, 5001
    x = g.normal(0.0, 0.1, (B, V)).astype(np.float32)
    _check(sampler, _wl(x, temperature=1.0, top_k=0, top_p=0.9))


@pytest.mark.parametrize("bf16", [False, True])
def test_window_sizes_either_side_of_the_shared_memory_tiers(sampler, bf16):
    """Rows with exactly m values inside the significance window, m stepping over the sizes at which
    the ordering changes method (rank sort up to 256, key network up to 2048, pair network up to 4096,
    global scratch above). Up to 4096 the row is decided in shared memory (no full-ordering flag)."""
    g = np.random.default_rng(77)
    V = 50257
    sizes = [255, 256, 257, 2047, 2048, 2049, 3000, 4095, 4096, 4097, 5000]
    x = np.full((len(sizes), V), -40.0, np.float32)
    for r, m in enumerate(sizes):
        at = g.choice(V, m, replace=False)
        x[r, at] = g.uniform(-12.0, 0.0, m).astype(np.float32)
        x[r, at[0]] = 0.0
    if bf16:
        x = narrow_bf16(x)
    for kw in (dict(top_p=0.9), dict(top_p=1.0, min_p=0.0005), dict(top_p=0.999)):
        w = _wl(x, temperature=1.0, top_k=0, **kw)
        gpu = parity.run_gpu(sampler, w, kept_capacity=64)
        orc = parity.run_oracle(w, oracle.EXP_CR, 64)
        assert np.array_equal(gpu.tokens, orc.tokens)
        assert np.array_equal(gpu.kept_count, orc.kept_count)
        assert np.array_equal(gpu.stats, orc.stats)
        for r, m in enumerate(sizes):
            assert bool(gpu.flags[r] & N.ROW_FULL_SORT) == (m > 4096), (m, hex(int(gpu.flags[r])))


@pytest.mark.parametrize("vocab", [50257, 128256])
def test_constant_and_two_level_rows_round_like_the_sequential_sums(sampler, vocab):
    """Rows of one repeated value, or two: every term of the long sums has the same bits, so whole runs of
    additions round the same way, land exactly between two floats again and again (the rounding then depends on
    the running sum's parity), and cross binades at known places: the sums, the cumulative cut and the
    walk must come out as the reference's left-to-right f32 chains, bit for bit."""
    g = np.random.default_rng(vocab)
    x = np.zeros((5, vocab), np.float32)
    x[1, :] = 3.25
    x[2, ::2] = np.float32(np.log(2.0))          # exponentials 1 and 1/2
    x[3, : vocab // 3] = 1.0
    x[4, :] = g.choice(np.array([0.0, 0.6931472, 1.3862944], np.float32), vocab)
    _check(sampler, _wl(x, temperature=1.0, top_k=0, top_p=0.9))
    _check(sampler, _wl(x, temperature=1.0, top_k=0, top_p=0.37, min_p=1e-7))
    _check(sampler, _wl(narrow_bf16(x), temperature=2.0, top_k=0, top_p=0.999))
