import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on the B200 box)")


@pytest.fixture(scope="session")
def sampler():
    """One CUDA sampler handle for the whole session; fails loudly without a GPU."""
    import scriptonait_b200 as sb
    s = sb.Sampler(device=0, max_batch=1024, max_vocab=262144, max_history=1024, max_top_k=1024)
    yield s
    s.close()
