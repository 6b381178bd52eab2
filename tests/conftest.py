import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(autouse=True)
def _reset_engine_config():
    from forgetrain_b200 import engine_config
    engine_config.reset_global_config()
    yield
    engine_config.reset_global_config()
