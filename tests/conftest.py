"""Test set-up: the `gpu` marker and the tiny model folders.

Tests marked `gpu` need a CUDA device (B200); all others run on the CPU.
Model folders are made in temporary folders, never in the repository.
"""
import os
import sys

import pytest

ROOT = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    config.addinivalue_line("markers", "slow: takes a minute or more (deselect with -m 'gpu and not slow')")


def pytest_collection_modifyitems(config, items):
    # the file whose name starts with test_zz runs last, whatever the order given
    items.sort(key=lambda item: os.path.basename(str(item.fspath)).startswith("test_zz"))


@pytest.fixture(scope="session")
def tiny_folders(tmp_path_factory):
    """{name: folder} for the two tiny configurations, written once per run."""
    import tiny
    root = tmp_path_factory.mktemp("models")
    return {name: tiny.write_folder(str(root / name), name) for name in tiny.CONFIGS}
