import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def cuda_runtime():
    """The product runtime over libdeepj_cuda_jni; fails loudly if the library is missing."""
    from deepj_b200.compute_graph import CudaGpuRuntime
    return CudaGpuRuntime(0)
