"""pytest configuration: registers the `gpu` marker and makes the repo importable.

`-m "not gpu"` tests run on a machine without a GPU: the oracle against the golden
vectors, host-side logic, and that the shared libraries load and export every symbol
the headers declare. `-m gpu` tests are the parity tests proper; they call the CUDA
path through the C ABI and compare it with the oracle / golden vectors.
"""
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


import pytest


@pytest.fixture(autouse=True)
def _release_scratch():
    yield
    try:
        from tests import pkt
        import torch
        if pkt._live and torch.cuda.is_available():
            pkt.release()
    except ImportError:
        pass
