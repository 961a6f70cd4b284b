"""Size-independent properties at the workloads' full sizes (no oracle in the loop):
determinism, idempotence over a read-only input, kept-set invariants, greedy == argmax,
row-permutation equivariance, split invariance, and the uniform-stream identity."""
import numpy as np
import pytest

import parity
from scriptonait_b200 import native as N
from scriptonait_b200 import workloads

pytestmark = pytest.mark.gpu


def test_c3_full_size_properties(sampler):
    import torch
    w = workloads.c3()
    lg = parity.device_logits(w)
    before = lg.view(torch.int16).clone()
    a = parity.run_gpu(sampler, w, logits_dev=lg)
    b = parity.run_gpu(sampler, w, logits_dev=lg)
    assert torch.equal(before, lg.view(torch.int16)), "the logits are read-only"
    assert np.array_equal(a.tokens, b.tokens) and np.array_equal(a.kept_probs, b.kept_probs)
    wide = workloads.widen_bf16(w.logits)
    mx = wide.max(axis=1)
    for r in range(w.batch):
        kc = int(a.kept_count[r])
        assert 1 <= kc <= 64
        ids = a.kept_ids[r, :kc]
        p = a.kept_probs[r, :kc]
        assert a.tokens[r] in ids
        assert (np.diff(p) <= 0).all()                       # most likely first
        assert (p >= np.float32(0.05) * p[0]).all()          # min-p invariant
        assert wide[r, ids[0]] == mx[r] and ids[0] == np.argmax(wide[r])   # leader = first index of the maximum
        assert a.stats[r, 1] >= 1.0 and 0 < a.stats[r, 2] <= 1.0 + 1e-6     # sum >= leader's 1, total <= 1
    # the uniform each row consumed is output 1 of SplitMix64(1234 + r)
    import scriptonait_b200 as sb
    for r in (0, 1, 100, 255):
        assert a.stats[r, 3] == np.float32(sb.Rng(1234 + r).next_f32())
    # permuting the rows (with their seeds) permutes the tokens
    perm = np.random.default_rng(0).permutation(w.batch)
    wp = workloads.row_slice(w, 0, w.batch)
    wp.logits, wp.seeds = w.logits[perm], w.seeds[perm]
    c = parity.run_gpu(sampler, wp)
    assert np.array_equal(c.tokens, a.tokens[perm])
    # the CTAs-per-row split is invisible in the result
    for split in (1, 2, 4):
        d = parity.run_gpu(sampler, w, logits_dev=lg, split=split)
        assert np.array_equal(d.tokens, a.tokens) and np.array_equal(d.kept_probs, a.kept_probs)


def test_c4_full_size_properties(sampler):
    w = workloads.c4(64)
    a = parity.run_gpu(sampler, w, kept_capacity=64)
    for r in range(0, w.batch, 7):
        kc = int(a.kept_count[r])
        assert 1 <= kc <= 64
        cum = np.cumsum(a.kept_probs[r, :kc].astype(np.float64))
        assert kc == 64 or cum[-1] >= 0.99 - 1e-6           # top-p cut reached, or everything kept
        assert kc == 1 or cum[-2] < 0.99 + 1e-6             # and not earlier
        assert a.tokens[r] in a.kept_ids[r, :kc]
    # top_k = 1 is greedy on the penalised row whatever the seed
    w1 = workloads.c4(1)
    b = parity.run_gpu(sampler, w1)
    w1g = workloads.c4(1)
    w1g.temperature = 0.0
    c = parity.run_gpu(sampler, w1g)
    assert np.array_equal(b.tokens, c.tokens)
    assert all(f & N.ROW_GREEDY for f in c.flags)


def test_greedy_equals_argmax_at_262144_columns(sampler):
    w = workloads.c5()
    w.temperature = 0.0
    a = parity.run_gpu(sampler, w)
    assert np.array_equal(a.tokens, np.argmax(w.logits, axis=1).astype(np.uint32))
