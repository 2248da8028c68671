import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


@pytest.fixture(autouse=True)
def _fresh_singletons():
    from crossbow_b200.conf import ModelConf, SystemConf
    SystemConf.reset()
    ModelConf.reset()
    yield
