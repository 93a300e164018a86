"""pytest configuration: registers the ``gpu`` marker and skips GPU tests without a device."""
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_addoption(parser):
    parser.addoption("--debug-bounds", action="store_true", default=False,
                     help="run against the checked-store build of the kernel library (every global store is "
                          "checked against the registered tensors; built on demand)")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")
    if config.getoption("--debug-bounds"):
        os.environ["DIZO_DEBUG_BOUNDS"] = "1"       # read when dizo_b200.ops._lib is first imported


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _run_in_scratch_directory(tmp_path, monkeypatch):
    """The trainer writes its ``loss_acc/`` curves and result files relative to the working directory,
    as the reference does (large_models/trainer.py:1331-1345); run every test from a scratch directory
    so that a test run leaves the source tree clean."""
    monkeypatch.chdir(tmp_path)
