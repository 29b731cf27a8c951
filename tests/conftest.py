"""Shared fixtures: the ``gpu`` marker, golden-vector loading, seeding."""

import glob
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu)")


def golden_names():
    return sorted(
        os.path.splitext(os.path.basename(p))[0]
        for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz"))
        if os.path.basename(p) != "step.npz" and not os.path.basename(p).startswith(("raw_", "decode_"))
    )


def load_golden(name):
    with np.load(os.path.join(GOLDEN_DIR, name + ".npz")) as z:
        return {k: z[k] for k in z.files}


@pytest.fixture(autouse=True)
def _seed():
    np.random.seed(0)
    try:
        import torch

        torch.manual_seed(0)
    except Exception:  # pragma: no cover
        pass
