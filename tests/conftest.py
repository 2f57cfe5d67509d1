import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run on a B200 box)")


@pytest.fixture(autouse=True)
def _reset_contexts():
    import mindspore_b200 as ms
    import torch
    ms.reset_auto_parallel_context()
    ms.set_context(mode=ms.PYNATIVE_MODE, device_target="GPU" if torch.cuda.is_available() else "CPU")
    yield
    ms.reset_auto_parallel_context()
