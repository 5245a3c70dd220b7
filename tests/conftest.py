import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def gpu():
    """The device handle every GPU test goes through. A GPU test without a
    device fails loudly: there is no CPU path to fall back to."""
    import torch

    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    from ttsxabe_b200 import Gpu

    g = Gpu.open(int(os.environ.get("LLMTIE_TEST_DEVICE", "0")))
    yield g
    g.synchronize()
