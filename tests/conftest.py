import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `-m gpu`)")
    # Make sure the shared library matches the sources; a no-op when it is up to date.
    from causal_tuner_b200 import build
    if not build.up_to_date():
        try:
            build.build()
        except Exception as error:  # no nvcc on this machine: the ABI tests will say so
            sys.stderr.write(f"libct_b200.so could not be rebuilt: {error}\n")


@pytest.fixture(autouse=True)
def reproducible():
    torch.manual_seed(4)
    torch.set_num_threads(max(1, min(8, os.cpu_count() or 1)))
    if torch.cuda.is_available():
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False


@pytest.fixture
def golden():
    import numpy as np

    def load(name):
        with np.load(os.path.join(GOLDEN, name)) as data:
            return {key: data[key] for key in data.files}
    return load


@pytest.fixture
def gpu_guard():
    """After a GPU test: synchronise and fail if a kernel reported a bounded-wait timeout."""
    yield
    from causal_tuner_b200 import _lib
    _lib.check_device()
