"""llm_cuda_cross_entropy against the oracle's restatement of llm_core::ops::cross_entropy
(crates/llm-core/src/ops/loss.rs:20-45). Floating point in a different summation order (the kernel reduces
in parallel, the reference left to right): the per-row loss must agree within 1e-5 relative to max(1, |loss|)
and every gradient entry within 1e-6 absolute (probabilities are at most 1; the tolerance the sampler's
probabilities are held to against the libm oracle)."""
import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


def _run(sampler, x, targets, want_grad=True, pad=0, offset=0):
    import torch
    t_len, vocab = x.shape
    if pad or offset:
        buf = torch.zeros(t_len * (vocab + pad) + offset + 8, dtype=torch.float32, device="cuda")
        lg = buf[offset: offset + t_len * (vocab + pad)].view(t_len, vocab + pad)[:, :vocab]
        lg.copy_(torch.from_numpy(x))
    else:
        lg = torch.from_numpy(x).cuda()
    tg = torch.from_numpy(np.asarray(targets, np.int32)).cuda()
    rows, grad = sampler.cross_entropy(lg, tg, want_grad=want_grad)
    torch.cuda.synchronize()
    return rows.cpu().numpy(), (grad.cpu().numpy() if want_grad else None)


def _check(sampler, x, targets, **kw):
    loss, d, rows = oracle.cross_entropy(x, targets)
    got_rows, got_d = _run(sampler, x, targets, **kw)
    assert np.abs(got_rows - rows).max() <= 1e-5 * max(1.0, float(np.abs(rows).max())), np.abs(got_rows - rows).max()
    assert np.abs(got_d - d).max() <= 1e-6, np.abs(got_d - d).max()
    assert abs(float(got_rows.astype(np.float64).mean()) - loss) <= 1e-5 * max(1.0, abs(loss))
    return got_rows, got_d


def test_reference_cases(sampler):
    # loss.rs:52-74 on the device: the uniform row, and a small matrix whose gradient rows sum to zero
    rows, d = _check(sampler, np.zeros((1, 10), np.float32), [3])
    assert abs(rows[0] - np.log(10.0)) < 1e-4
    g = np.random.default_rng(70)
    x = g.normal(0, 1, (3, 6)).astype(np.float32)
    rows, d = _check(sampler, x, [1, 4, 0])
    assert (rows > 0).all() and np.abs(d.sum(axis=1)).max() < 1e-6


@pytest.mark.parametrize("t_len,vocab", [(1, 1), (2, 3), (5, 4096), (256, 4096), (7, 50257), (64, 128256)])
def test_shapes_from_the_reference_scale_to_128k(sampler, t_len, vocab):
    g = np.random.default_rng(vocab + t_len)
    x = g.normal(0.0, 2.5, (t_len, vocab)).astype(np.float32)
    targets = g.integers(0, vocab, t_len)
    targets[0] = int(np.argmax(x[0]))          # the target is the leader
    targets[-1] = int(np.argmin(x[-1]))        # ... and the least likely id
    _check(sampler, x, targets)


def test_rows_that_do_not_start_on_16_bytes_and_padded_strides(sampler):
    g = np.random.default_rng(9)
    x = g.normal(0.0, 1.0, (6, 1003)).astype(np.float32)
    targets = g.integers(0, 1003, 6)
    for pad, offset in ((0, 1), (5, 0), (2, 3), (1, 2)):
        _check(sampler, x, targets, pad=pad, offset=offset)


def test_peaked_and_masked_rows(sampler):
    g = np.random.default_rng(10)
    x = g.normal(0.0, 1.0, (4, 5000)).astype(np.float32)
    x[0, 17] = 80.0                            # one id takes everything: the others' exponentials underflow
    x[1, ::2] = -np.inf                        # masked ids contribute nothing and get gradient zero
    x[2, :] = -1e4
    x[3, :100] = 30.0
    targets = [17, 1, 4999, 50]
    _check(sampler, x, targets)


def test_loss_only_and_bad_arguments(sampler):
    import torch
    from scriptonait_b200 import native as N
    g = np.random.default_rng(11)
    x = g.normal(0.0, 1.0, (3, 777)).astype(np.float32)
    rows, none = _run(sampler, x, [0, 1, 2], want_grad=False)
    assert none is None and np.abs(rows - oracle.cross_entropy(x, [0, 1, 2])[2]).max() < 1e-5
    # a target outside the vocabulary (the reference panics): that row's loss is NaN, nothing is read out of bounds
    rows, d = _run(sampler, x, [0, 777, 2])
    assert np.isnan(rows[1]) and np.isfinite(rows[[0, 2]]).all() and np.isfinite(d).all()
    with pytest.raises(ValueError):
        sampler.cross_entropy(torch.zeros((2, 8), dtype=torch.float16, device="cuda"), torch.zeros(2, dtype=torch.int32, device="cuda"))
