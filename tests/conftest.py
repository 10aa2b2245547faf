"""Shared test plumbing: import paths, the ``gpu`` marker, golden-file access."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests", "golden")):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    # GPU tests are selected with `-m gpu`; without a device they are skipped, not failed.
    try:
        import torch
        have = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        have = False
    if have:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


class Golden:
    """Grouped view of an ``.npz`` whose keys look like ``case/field``."""

    def __init__(self, name):
        self.z = np.load(os.path.join(GOLDEN, name))
        self.cases = sorted({k.split("/")[0] for k in self.z.files})

    def case(self, name):
        return {k.split("/", 1)[1]: self.z[k] for k in self.z.files if k.startswith(name + "/")}


@pytest.fixture(scope="session")
def golden_token():
    return Golden("token_cases.npz")


@pytest.fixture(scope="session")
def golden_logits():
    return Golden("logits_cases.npz")


@pytest.fixture(scope="session")
def golden_fixtures():
    return Golden("reference_fixtures.npz")
