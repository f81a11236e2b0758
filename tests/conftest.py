"""pytest configuration: the `gpu` marker, repository root on sys.path, golden-fixture loader."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box only)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        have_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        have_gpu = False
    if have_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device visible")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


GOLDEN_CASES = ["len1", "len2", "odd17", "pow64", "batch3d", "ragged300", "slow1000", "slower2100"]


@pytest.fixture(scope="session")
def golden():
    path = os.path.join(ROOT, "tests", "golden", "linrec_golden.npz")
    with np.load(path) as z:
        return {k: z[k] for k in z.files}
