"""Shared test setup: the `gpu` marker, import paths and golden-vector loading."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")
for path in (ROOT, GOLDEN):
    if path not in sys.path:
        sys.path.insert(0, path)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    with np.load(os.path.join(GOLDEN, name + ".npz")) as data:
        return {k: data[k] for k in data.files}


@pytest.fixture(scope="session")
def native():
    """The built C-ABI library wrapper (building it first if the .so is absent)."""
    from gl_sdm_b200 import _native
    if not os.path.exists(_native.LIBRARY_PATH):
        import __graft_entry__
        __graft_entry__.build()
    _native.library()
    return _native
