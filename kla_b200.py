"""Import alias: ``import kla_b200`` gives the package in the directory
``kalman-linear-attention_b200`` (whose name is not a Python identifier)."""

import importlib
import os
import sys

_root = os.path.dirname(os.path.abspath(__file__))
if _root not in sys.path:
    sys.path.insert(0, _root)
sys.modules[__name__] = importlib.import_module("kalman-linear-attention_b200")
