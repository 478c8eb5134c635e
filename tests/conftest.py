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
def oracle():
    from oracle import q4_oracle

    q4_oracle.build()
    return q4_oracle


@pytest.fixture(scope="session")
def golden():
    import json

    with open(os.path.join(ROOT, "tests", "golden", "reference_cases.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def runtime():
    """One CudaRuntime for the GPU tests. Building is a no-op when lib/libq4b200.so is current."""
    from qwen38_metal_b200 import build, runtime as rt_mod

    build.build()
    rt = rt_mod.CudaRuntime(0)
    yield rt
    rt.close()
