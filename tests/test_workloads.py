"""The synthetic workload generators: shapes, dtypes, determinism and the distributions'
fingerprints the parity and bench runs rely on."""
import numpy as np

from scriptonait_b200 import workloads


def test_shapes_and_algorithmic_bytes():
    w1 = workloads.c1(1000)
    assert w1.logits.shape == (1, 8192) and w1.batch == 1000 and w1.history.shape == (1000, 64) and w1.broadcast_row
    assert w1.algorithmic_bytes() // 1000 == 33028
    w2 = workloads.c2()
    assert w2.logits.shape == (64, 32768) and w2.algorithmic_bytes() == 8454400
    w4 = workloads.c4(8, batch=16)
    assert w4.logits.shape == (16, 50257) and w4.history.shape == (16, 512)
    assert workloads.Workload("x", np.zeros((256, 128256), np.uint16), batch=256).algorithmic_bytes() == 65668096
    assert workloads.Workload("x", np.zeros((1024, 50257), np.float32), history=np.zeros((1024, 512), np.uint32),
                              batch=1024).algorithmic_bytes() == 207953920
    assert workloads.Workload("x", np.zeros((32, 262144), np.float32), batch=32).algorithmic_bytes() == 33554560


def test_generators_are_deterministic_and_seeded_per_row():
    a, b = workloads.c3(batch=4, vocab=4096), workloads.c3(batch=4, vocab=4096)
    assert np.array_equal(a.logits, b.logits) and a.logits.dtype == np.uint16
    assert not np.array_equal(a.logits, workloads.c3(batch=4, vocab=4096, variant=1).logits)
    assert list(a.seeds) == [1234, 1235, 1236, 1237]
    assert list(workloads.c3(batch=2, vocab=1024, row0=10).seeds) == [1244, 1245]


def test_c3_is_zipf_peaked_and_c5_has_masked_entries_and_c1_has_boosts():
    w = workloads.c3(batch=2, vocab=128256)
    wide = workloads.widen_bf16(w.logits)
    assert ((wide.max(axis=1, keepdims=True) - wide) <= 17.4).sum(axis=1).max() < 1000
    w5 = workloads.c5(batch=2, vocab=65536)
    frac = np.isneginf(w5.logits).mean()
    assert 0.005 < frac < 0.015
    w1 = workloads.c1(3)
    assert (w1.logits[0] > 8).sum() <= 8 and w1.logits[0].max() > 4


def test_row_slice_keeps_rows_params_and_seeds_together():
    w = workloads.c2(batch=8, vocab=1024, hist_len=16)
    s = workloads.row_slice(w, 2, 5)
    assert s.batch == 3 and np.array_equal(s.logits, w.logits[2:5]) and np.array_equal(s.temperature, w.temperature[2:5])
    assert np.array_equal(s.history, w.history[2:5]) and list(s.seeds) == [1236, 1237, 1238]
