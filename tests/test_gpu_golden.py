"""The CUDA path against the committed golden vectors (no oracle in the loop): bit for bit
against the vectors written with the correctly rounded exp, within the stated tolerance
against the ones written with the generating host's expf."""
import pytest

import golden_io
import parity

pytestmark = pytest.mark.gpu
CASES = golden_io.load()


@pytest.mark.parametrize("name", sorted(CASES))
def test_cuda_path_reproduces_the_golden_vectors(sampler, name):
    w, frozen = CASES[name]
    gpu = parity.run_gpu(sampler, w, kept_capacity=64)
    parity.assert_exact(parity.compare(frozen["cr"], gpu, w, exact=True))
    parity.assert_within_tolerance(parity.compare(frozen["libm"], gpu, w, exact=False))
