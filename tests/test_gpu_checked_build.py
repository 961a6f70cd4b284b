"""The bounds-checked build of the library (the same sources with -DLLM_CUDA_CHECKED) on small, odd and
awkward shapes: every store at a computed shared-memory or scratch offset is compared with its region's
size first, and a violation sets LLM_CUDA_STATUS_CHECK_FAILED in the device status word (the store is
skipped, nothing traps). Every case must match the oracle bit for bit AND leave the status word at 0.
This stands in for compute-sanitizer, which is closed on this pool."""
import numpy as np
import pytest

import oracle
import parity
from scriptonait_b200.workloads import Workload, narrow_bf16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def checked():
    import scriptonait_b200 as sb
    s = sb.Sampler(device=0, max_batch=64, max_vocab=140000, max_history=1024, max_top_k=2048, checked=True)
    yield s
    s.close()


def _run(checked, w, kept_capacity=64, allowed=None, **kw):
    gpu = parity.run_gpu(checked, w, kept_capacity=kept_capacity, allowed=allowed, **kw)
    rep = parity.compare(parity.run_oracle(w, oracle.EXP_CR, kept_capacity, allowed=allowed), gpu, w, exact=True)
    parity.assert_exact(rep)
    assert checked.device_status() == 0, "an index check failed in the checked build"


def _wl(x, **kw):
    B = x.shape[0]
    kw.setdefault("seeds", np.arange(B, dtype=np.uint64) + np.uint64(77))
    return Workload("checked", x, batch=B, **kw)


@pytest.mark.parametrize("V", [1, 3, 4, 5, 31, 33, 257, 1023, 4097, 12289, 50257])
@pytest.mark.parametrize("bf16", [False, True])
def test_odd_vocabulary_sizes(checked, V, bf16):
    g = np.random.default_rng(V)
    x = g.normal(0, 2, (5, V)).astype(np.float32)
    hist = g.integers(0, V + 3, size=(5, 40), dtype=np.uint32)
    if bf16:
        x = narrow_bf16(x)
    _run(checked, _wl(x, temperature=0.8, top_k=min(40, V), top_p=0.95, min_p=0.01, repetition_penalty=1.2, history=hist))
    _run(checked, _wl(x, temperature=1.0, top_k=0, top_p=1.0, min_p=0.05))  # window rows


@pytest.mark.parametrize("top_k", [1, 255, 256, 257, 1024, 2048])
def test_every_rank_cut_class_with_long_history(checked, top_k):
    g = np.random.default_rng(top_k)
    V = 30011
    x = g.normal(0, 1.5, (4, V)).astype(np.float32)
    hist = g.integers(0, V, size=(4, 1024), dtype=np.uint32)
    _run(checked, _wl(x, temperature=0.9, top_k=top_k, top_p=0.97, repetition_penalty=1.3, history=hist), kept_capacity=128)


@pytest.mark.parametrize("split", [1, 2, 5])
def test_split_rows_masks_and_misaligned_rows(checked, split):
    g = np.random.default_rng(3 + split)
    V = 50257                                        # rows only 4-byte aligned
    x = g.normal(0, 0.5, (6, V)).astype(np.float32)
    allowed = g.random(V) < 0.5
    hist = g.integers(0, V, size=(6, 300), dtype=np.uint32)
    _run(checked, _wl(x, temperature=1.0, top_k=64, top_p=0.99, repetition_penalty=1.3, history=hist), allowed=allowed,
         split=split)


def test_ascending_rows_and_window_overflow_into_the_full_ordering(checked):
    V = 20000
    base = np.linspace(-8.0, 8.0, V, dtype=np.float32)
    x = np.stack([base, base[::-1].copy()])
    _run(checked, _wl(x, temperature=0.9, top_k=300, top_p=0.97), kept_capacity=128)
    flat = np.random.default_rng(1).normal(0, 0.2, (3, 9000)).astype(np.float32)   # every value inside the window
    _run(checked, _wl(flat, temperature=1.0, top_k=0, top_p=0.9))
