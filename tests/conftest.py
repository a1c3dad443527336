"""Shared fixtures.  ``-m gpu`` tests need a CUDA device; everything else runs on CPU."""
import gzip
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name: str):
    with gzip.open(os.path.join(GOLDEN, f"{name}.pt.gz"), "rb") as fh:
        return torch.load(fh, weights_only=False)


@pytest.fixture(scope="session")
def golden_tables():
    return load_golden("tables")


@pytest.fixture(scope="session")
def golden_ops():
    return load_golden("ops")


@pytest.fixture(scope="session")
def golden_layers():
    return load_golden("layers")
