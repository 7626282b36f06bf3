import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
if os.path.dirname(os.path.abspath(__file__)) not in sys.path:
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def tiny_folders(tmp_path_factory):
    """Model folders of the tiny configurations, written once per session in a temporary place."""
    from helpers import TINY_CONFIGS, make_folder

    root = tmp_path_factory.mktemp("tiny_models")
    return {name: make_folder(root / name, name) for name in TINY_CONFIGS}
