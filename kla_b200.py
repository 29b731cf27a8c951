"""Import alias: ``import kla_b200`` gives the package in the directory
``kalman-linear-attention_b200`` (whose name is not a Python identifier).

Run as a script it is the reference's command line with the ``b200`` backend in
its tables: ``python kla_b200.py --check-backends`` (see the package's ``cli.py``)."""

import importlib
import os
import sys

_root = os.path.dirname(os.path.abspath(__file__))
if _root not in sys.path:
    sys.path.insert(0, _root)
_pkg = importlib.import_module("kalman-linear-attention_b200")
if __name__ == "__main__":
    sys.modules["kla_b200"] = _pkg
    raise SystemExit(importlib.import_module("kalman-linear-attention_b200.cli").main())
sys.modules[__name__] = _pkg
