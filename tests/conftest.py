import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `-m gpu`)")
    config.addinivalue_line("markers", "slow: multi-process or long-running test")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def cuda_status():
    """Yields the device status word and asserts afterwards that no kernel wait timed out."""
    from forgeminds_b200 import ops
    word = ops.status_word("cuda")
    word.zero_()
    yield word
    assert int(word.item()) == 0, "a kernel reported a timed-out wait"
