"""The oracle's cross-entropy (a restatement of llm_core::ops::cross_entropy, crates/llm-core/src/ops/loss.rs:20-45)
against the reference's own two tests of it (loss.rs:52-74) and against float64 arithmetic."""
import numpy as np

import oracle


def _seeded(seed, n):
    g = np.random.default_rng(seed)
    return g.normal(0.0, 1.0, n).astype(np.float32)


def test_gradient_matches_finite_differences():
    # loss.rs:53-65: T = 3, vocab = 6, targets [1, 4, 0], central differences with step 1e-3, tolerance 1e-3
    t_len, vocab = 3, 6
    x = _seeded(70, t_len * vocab).reshape(t_len, vocab)
    targets = [1, 4, 0]
    loss, d, _ = oracle.cross_entropy(x, targets)
    assert loss > 0.0
    num = np.zeros_like(x)
    for i in range(t_len):
        for j in range(vocab):
            hi = x.copy(); hi[i, j] += 1e-3
            lo = x.copy(); lo[i, j] -= 1e-3
            num[i, j] = (oracle.cross_entropy(hi, targets, want_grad=False)[0] - oracle.cross_entropy(lo, targets, want_grad=False)[0]) / 2e-3
    assert np.abs(d - num).max() < 1e-3


def test_uniform_prediction_gives_log_vocab():
    # loss.rs:67-74
    loss, _, _ = oracle.cross_entropy(np.zeros((1, 10), np.float32), [3])
    assert abs(loss - np.log(10.0)) < 1e-4


def test_against_float64():
    g = np.random.default_rng(5)
    x = g.normal(0.0, 3.0, (7, 4096)).astype(np.float32)
    targets = g.integers(0, 4096, 7)
    loss, d, rows = oracle.cross_entropy(x, targets)
    w = x.astype(np.float64)
    lse = np.log(np.exp(w - w.max(axis=1, keepdims=True)).sum(axis=1)) + w.max(axis=1)
    want_rows = lse - w[np.arange(7), targets]
    assert np.abs(rows - want_rows).max() < 1e-4
    assert abs(loss - want_rows.mean()) < 1e-4
    p = np.exp(w - lse[:, None])
    p[np.arange(7), targets] -= 1.0
    assert np.abs(d - p / 7).max() < 1e-6
    assert np.abs(d.sum(axis=1)).max() < 1e-5   # a softmax minus a one-hot sums to zero
