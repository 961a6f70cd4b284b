"""Edge cases of the CUDA path against the oracle (bit-exact bar, correctly rounded exp):
tiny and ragged vocabularies, misaligned rows, top_k >= vocab, empty and duplicate-heavy
histories, ids outside the vocabulary, greedy rows, -inf / +inf rows, the allowed mask
with the EOS exemption, per-row parameter arrays, split rows, and the full-sort kernel."""
import numpy as np
import pytest

import oracle
import parity
from scriptonait_b200 import native as N
from scriptonait_b200.workloads import Workload, narrow_bf16

pytestmark = pytest.mark.gpu
INF = np.float32(np.inf)


def _wl(logits, **kw):
    B = logits.shape[0]
    kw.setdefault("seeds", np.arange(B, dtype=np.uint64) + np.uint64(77))
    return Workload("edge", logits, batch=B, **kw)


def _check(sampler, w, kept_capacity=64, allowed=None, **kw):
    gpu = parity.run_gpu(sampler, w, kept_capacity=kept_capacity, allowed=allowed, **kw)
    rep = parity.compare(parity.run_oracle(w, oracle.EXP_CR, kept_capacity, allowed=allowed), gpu, w, exact=True)
    parity.assert_exact(rep)
    return gpu, rep


@pytest.mark.parametrize("vocab", [1, 2, 3, 5, 31, 33, 255, 257, 1000, 4095, 4097, 8191, 12289, 50257])
@pytest.mark.parametrize("bf16", [False, True])
def test_ragged_vocab_sizes_and_misaligned_rows(sampler, vocab, bf16):
    g = np.random.default_rng(vocab)
    B = 9
    x = g.normal(0, 2.5, (B, vocab)).astype(np.float32)
    logits = narrow_bf16(x) if bf16 else x
    hist = g.integers(0, vocab + 2, size=(B, 17), dtype=np.uint32)
    w = _wl(logits, temperature=0.9, top_k=40, top_p=0.95, min_p=0.02, repetition_penalty=1.2, history=hist)
    _check(sampler, w)


@pytest.mark.parametrize("offset", [1, 2, 3, 5, 7])
def test_logits_pointer_not_16_byte_aligned(sampler, offset):
    import torch
    g = np.random.default_rng(offset)
    B, V = 6, 5003
    x = g.normal(0, 2, (B, V)).astype(np.float32)
    flat = torch.zeros(B * V + 16, dtype=torch.float32, device="cuda:0")
    view = flat[offset:offset + B * V].view(B, V)
    view.copy_(torch.from_numpy(x))
    w = _wl(x, temperature=1.1, top_k=12, top_p=0.9)
    gpu = parity.run_gpu(sampler, w, logits_dev=view)
    parity.assert_exact(parity.compare(parity.run_oracle(w, oracle.EXP_CR), gpu, w, exact=True))


def test_top_k_larger_than_vocab_and_top_k_zero_small_vocab(sampler):
    g = np.random.default_rng(1)
    x = g.normal(0, 1, (8, 37)).astype(np.float32)
    _check(sampler, _wl(x, temperature=1.0, top_k=1000, top_p=0.9))
    _check(sampler, _wl(x, temperature=1.0, top_k=0, top_p=1.0))
    _check(sampler, _wl(x, temperature=0.7, top_k=37, min_p=0.1))


def test_greedy_rows_after_penalty_and_first_index_ties(sampler):
    x = np.array([[2.0, 1.9, 0.0, 2.0], [1.0, 3.0, 3.0, -1.0], [-INF, -INF, -INF, -INF], [0.0, -0.0, -1.0, 0.0]], np.float32)
    hist = np.array([[0, 0], [9, 9], [1, 1], [3, 2]], np.uint32)
    w = _wl(x, temperature=0.0, repetition_penalty=1.5, history=hist)
    gpu, _ = _check(sampler, w)
    assert list(gpu.tokens) == [3, 1, 0, 0]
    assert all(f & N.ROW_GREEDY and not f & N.ROW_DRAW_CONSUMED for f in gpu.flags)


def test_duplicate_heavy_history_compounds_per_occurrence(sampler):
    g = np.random.default_rng(2)
    B, V = 16, 3000
    x = g.normal(0, 2, (B, V)).astype(np.float32)
    hist = g.integers(0, 40, size=(B, 300), dtype=np.uint32)  # ~7 repeats per id
    hist[:, ::7] = g.integers(V, V + 1000, size=hist[:, ::7].shape)  # ids past the vocabulary are skipped
    _check(sampler, _wl(x, temperature=0.8, top_k=50, top_p=0.95, repetition_penalty=1.3, history=hist))
    _check(sampler, _wl(x, temperature=0.8, top_k=50, top_p=0.95, repetition_penalty=0.7, history=hist))


def test_all_neg_inf_and_pos_inf_rows_are_degenerate(sampler):
    x = np.zeros((4, 300), np.float32)
    x[0, :] = -INF
    x[1, :] = -INF
    x[1, 17] = 2.0
    x[2, 5] = INF
    x[2, 100] = INF
    x[3, :] = np.linspace(-3, 3, 300, dtype=np.float32)
    for k in (0, 10):
        gpu, _ = _check(sampler, _wl(x, temperature=1.0, top_k=k, top_p=0.9))
        assert gpu.tokens[0] == 0 and gpu.flags[0] & N.ROW_DEGENERATE
        assert gpu.tokens[1] == 17
        assert gpu.tokens[2] == 5 and gpu.flags[2] & N.ROW_DEGENERATE


def test_allowed_mask_with_eos_exemption_and_short_mask(sampler):
    g = np.random.default_rng(3)
    B, V = 12, 2000
    x = g.normal(0, 2, (B, V)).astype(np.float32)
    x[:, 258] += 3.0
    allowed = g.random(1777) < 0.5
    allowed[258] = False
    w = _wl(x, temperature=1.0, top_k=30, top_p=0.95, repetition_penalty=1.1,
            history=g.integers(0, V, size=(B, 64), dtype=np.uint32))
    gpu, _ = _check(sampler, w, allowed=allowed)
    blocked = set(np.nonzero(~allowed)[0]) - {258}
    assert not (set(gpu.tokens.tolist()) & blocked)
    wg = _wl(x, temperature=0.0)
    _check(sampler, wg, allowed=allowed)


def test_per_row_parameter_arrays_mix_modes_in_one_launch(sampler):
    g = np.random.default_rng(4)
    B, V = 32, 9000
    x = g.normal(0, 2, (B, V)).astype(np.float32)
    w = _wl(x, temperature=g.choice([0.0, 0.6, 1.0, 1.4], B).astype(np.float32),
            top_k=g.choice([0, 1, 5, 40, 500, 20000], B).astype(np.uint32),
            top_p=g.choice([1.0, 0.9, 0.5], B).astype(np.float32),
            min_p=g.choice([0.0, 0.05, 2.0], B).astype(np.float32),
            repetition_penalty=g.choice([1.0, 1.2], B).astype(np.float32),
            history=g.integers(0, V, size=(B, 50), dtype=np.uint32))
    _check(sampler, w)


@pytest.mark.parametrize("split", [2, 5, 16])
def test_rows_split_over_several_ctas(sampler, split):
    g = np.random.default_rng(5)
    B, V = 7, 70001
    x = g.normal(0, 2, (B, V)).astype(np.float32)
    hist = g.integers(0, V, size=(B, 128), dtype=np.uint32)
    _check(sampler, _wl(x, temperature=0.9, top_k=64, top_p=0.92, repetition_penalty=1.15, history=hist), split=split)
    _check(sampler, _wl(narrow_bf16(x), temperature=1.0, top_k=0, min_p=0.03), split=split)
    _check(sampler, _wl(x, temperature=0.0), split=split)


def test_full_sort_kernel_agrees_with_the_streaming_path(sampler):
    g = np.random.default_rng(6)
    B, V = 10, 6001
    x = g.normal(0, 2, (B, V)).astype(np.float32)
    hist = g.integers(0, V, size=(B, 30), dtype=np.uint32)
    w = _wl(x, temperature=0.8, top_k=25, top_p=0.9, min_p=0.01, repetition_penalty=1.25, history=hist)
    gpu, _ = _check(sampler, w, force_full_sort=True)
    assert all(f & N.ROW_FULL_SORT for f in gpu.flags)
    w2 = _wl(x, temperature=0.0, repetition_penalty=1.25, history=hist)
    _check(sampler, w2, force_full_sort=True)


def test_flat_distribution_without_truncation_overflows_the_window_and_is_resolved_exactly(sampler):
    """Temperature-only sampling of a near-flat row keeps every id: the window cannot hold
    them, so the full-sort kernel must produce the reference's answer."""
    g = np.random.default_rng(7)
    B, V = 4, 20000
    x = g.normal(0, 0.2, (B, V)).astype(np.float32)
    w = _wl(x, temperature=1.0, top_k=0, top_p=1.0, min_p=0.0)
    gpu = parity.run_gpu(sampler, w)
    orc = parity.run_oracle(w, oracle.EXP_CR)
    assert np.array_equal(gpu.tokens, orc.tokens)
    assert np.array_equal(gpu.kept_count, orc.kept_count)
    assert all(f & N.ROW_FULL_SORT for f in gpu.flags)
    assert np.array_equal(gpu.stats, orc.stats)


def test_peaked_distribution_without_truncation_stays_on_the_window_path(sampler):
    g = np.random.default_rng(8)
    B, V = 16, 30000
    x = g.normal(0, 4.0, (B, V)).astype(np.float32)
    x[np.arange(B), g.integers(0, V, B)] = 34.0  # the rest tops out near 16: a few dozen values fall inside the window
    w = _wl(x, temperature=1.0, top_k=0, top_p=1.0, min_p=0.0)
    gpu = parity.run_gpu(sampler, w)
    orc = parity.run_oracle(w, oracle.EXP_CR)
    assert np.array_equal(gpu.tokens, orc.tokens)
    assert np.array_equal(gpu.kept_count, orc.kept_count)  # = vocab: nothing is cut
    assert np.array_equal(gpu.stats, orc.stats)
    assert all(f & N.ROW_WINDOWED for f in gpu.flags)


def test_uniform_override_pins_the_stream(sampler):
    g = np.random.default_rng(9)
    B, V = 8, 1000
    x = g.normal(0, 2, (B, V)).astype(np.float32)
    w = _wl(x, temperature=1.0, top_k=10)
    u = np.full(B, 0.0, np.float32)
    gpu = parity.run_gpu(sampler, w, uniforms=u)
    assert np.array_equal(gpu.tokens, np.argmax(x, axis=1).astype(np.uint32))  # u = 0 picks the leader
    u1 = np.full(B, np.float32(1.0) - np.float32(2 ** -24), np.float32)
    gpu = parity.run_gpu(sampler, w, uniforms=u1)
    order = np.argsort(-x, axis=1, kind="stable")[:, :10]
    assert all(gpu.tokens[r] in order[r, -2:] for r in range(B))


def test_invalid_arguments_are_reported_not_raised_from_the_gpu(sampler):
    import torch
    import scriptonait_b200 as sb
    x = torch.zeros((2, 10), dtype=torch.float32, device="cuda:0")
    with pytest.raises(sb.LlmCudaError) as e:
        sampler.sample_batch(x, temperature=float("nan"))
    assert e.value.code == N.ERR_BAD_ARGUMENT
    big = torch.zeros((2, 10), dtype=torch.float32, device="cuda:0")
    with pytest.raises(sb.LlmCudaError) as e:
        sampler.sample_batch(big, batch=5000)
    assert e.value.code == N.ERR_CAPACITY
    res = sampler.sample_batch(x, temperature=torch.tensor([float("nan"), 1.0]), trace=True)
    torch.cuda.synchronize()
    assert int(res.row_flags[0]) & N.ROW_INVALID and int(res.tokens[0]) == 0
