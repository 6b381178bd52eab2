import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    """GPU tests are skipped on a machine without a CUDA device. With one, every GPU test gets a
    hard time limit (when pytest-timeout is installed): a device-side wait that never ends blocks
    the host inside the CUDA runtime, where only a watchdog thread that ends the process can
    still act."""
    import torch
    if not torch.cuda.is_available():
        # a machine without a CUDA device: GPU tests are skipped, not failed. (With a device they
        # run, and fail loudly if the native library cannot be loaded: nothing is skipped there.)
        skip = pytest.mark.skip(reason="needs a CUDA device")
        for item in items:
            if item.get_closest_marker("gpu"):
                item.add_marker(skip)
    if not config.pluginmanager.hasplugin("timeout"):
        return
    for item in items:
        if item.get_closest_marker("gpu") and not item.get_closest_marker("timeout"):
            item.add_marker(pytest.mark.timeout(240, method="thread"))


@pytest.fixture(autouse=True)
def _reset_engine_config():
    from forgetrain_b200 import engine_config
    engine_config.reset_global_config()
    yield
    engine_config.reset_global_config()
