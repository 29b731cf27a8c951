"""``python -m kla`` with the ``b200`` backend in its tables.

The reference's command line lists, probes and tests the scan backends
(``python -m kla --check-backends`` / ``--test-backends NAME``,
src/kla/__main__.py). Its tables are plain module-level dicts and a function:
``_DESCRIPTIONS`` and ``_MODULES`` (:30-42) and ``_requirements()`` (:104-133).
``main()`` here registers the backend (see ``register.py``), adds the ``b200``
rows to those three, and hands over to the reference's own ``main`` -- nothing in
the reference is edited, and its checks (``_forward``, ``_gradients``) run the
B200 kernels against ``kla_scan_reference`` exactly as they run the other backends.

    python kla_b200.py --check-backends
    python kla_b200.py --test-backends b200

The accuracy budget the reference prints for every backend (atol = rtol = 5e-4,
gradients 1e-2 of scale, :62-63) applies unchanged; the ``b200`` gradients are exact
for all six inputs, so no entry in ``_LOOSE_GRADS`` is added.
"""

from __future__ import annotations

import os

from . import _lib
from .register import register

DESCRIPTION = "hand-written sm_100a kernels for B200; exact gradients, state in and out"


def install_rows(name: str = "b200") -> None:
    """Add the backend's rows to the reference CLI's tables (idempotent)."""
    import kla.__main__ as kla_main

    kla_main._DESCRIPTIONS[name] = DESCRIPTION
    kla_main._MODULES[name] = "kla_b200"
    if getattr(kla_main._requirements, "_kla_b200", False):
        return
    inner = kla_main._requirements

    def _requirements():
        import torch

        rows = inner()
        sm100 = torch.cuda.is_available() and torch.cuda.get_device_capability(0)[0] == 10
        rows[name] = [
            (torch.cuda.is_available(), "needs a CUDA device"),
            (sm100, "needs an sm_100 GPU (B200)"),
            (os.path.exists(_lib.LIB_PATH),
             "needs libkla_b200.so: python kalman-linear-attention_b200/build.py"),
        ]
        return rows

    _requirements._kla_b200 = True
    kla_main._requirements = _requirements


def main(argv=None) -> int:
    import tyro
    import kla.__main__ as kla_main

    register()
    install_rows()
    return tyro.cli(kla_main.main, prog="python kla_b200.py", args=argv)
