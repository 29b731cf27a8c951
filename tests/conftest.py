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


def reference_src() -> str:
    """Directory that holds the reference package ``kla``: ``$KLA_REFERENCE_SRC`` when set, else the copy
    ``baseline/install_reference.py`` leaves under ``baseline/_ref``; "" when neither exists (tests then skip)."""
    cand = os.environ.get("KLA_REFERENCE_SRC") or os.path.join(ROOT, "baseline", "_ref")
    return cand if os.path.isfile(os.path.join(cand, "kla", "__init__.py")) else ""


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
