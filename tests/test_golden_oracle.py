"""The committed golden vectors (tests/golden/sampler_cases.npz, written by
tests/golden/make_golden.py) against the oracle as built on this machine: bit for bit
under the correctly rounded exp; under this host's expf within the stated tolerance (the C
library may differ from the one that wrote the file)."""
import numpy as np
import pytest

import golden_io
import oracle
import parity

CASES = golden_io.load()


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_reproduces_the_golden_vectors_bit_for_bit_with_correctly_rounded_exp(name):
    w, frozen = CASES[name]
    now = parity.run_oracle(w, oracle.EXP_CR, kept_capacity=64, threads=1)
    f = frozen["cr"]
    assert np.array_equal(now.tokens, f.tokens)
    assert np.array_equal(now.flags, f.flags)
    assert np.array_equal(now.kept_count, f.kept_count)
    assert np.array_equal(now.kept_ids, f.kept_ids)
    assert np.array_equal(now.kept_probs.view(np.uint32), f.kept_probs.view(np.uint32))
    assert np.array_equal(now.stats.view(np.uint32), f.stats.view(np.uint32))


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_with_the_host_expf_stays_within_tolerance_of_the_golden_vectors(name):
    w, frozen = CASES[name]
    now = parity.run_oracle(w, oracle.EXP_LIBM, kept_capacity=64, threads=1)
    as_gpu = parity.GpuOut(now.tokens, now.flags, now.kept_count, now.kept_ids, now.kept_probs, now.stats)
    rep = parity.compare(frozen["libm"], as_gpu, w, exact=False)
    parity.assert_within_tolerance(rep)


def test_golden_file_covers_every_stage():
    flags = np.concatenate([f["cr"].flags for _, f in CASES.values()])
    assert (flags & oracle.FLAG_GREEDY).any() and (flags & oracle.FLAG_DEGENERATE).any() and (flags & oracle.FLAG_DRAW_CONSUMED).any()
    kept = np.concatenate([f["cr"].kept_count for _, f in CASES.values()])
    assert kept.max() > 40 and (kept == 1).any()
