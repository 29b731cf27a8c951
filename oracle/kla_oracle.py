"""ctypes binding of the C oracle (``oracle/kla_oracle.c``).

TEST INFRASTRUCTURE ONLY. The oracle restates the reference's sequential
filter (``src/kla/ops/kla_ops.py:293-362``) and its exact adjoint on the CPU.
It is the checker for the parity tests, for the smoke check, and the thing
timed as the CPU baseline; the product path never imports it.

Arrays are numpy, C-contiguous, float64 (default) or float32; the dtype picks
the ``_f64`` / ``_f32`` entry points.
"""

from __future__ import annotations

import ctypes
import os
import subprocess
from typing import NamedTuple, Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libkla_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile ``libkla_oracle.so`` with the Makefile beside this file."""
    src_newer = os.path.exists(_LIB_PATH) and any(
        os.path.getmtime(os.path.join(_HERE, f)) > os.path.getmtime(_LIB_PATH)
        for f in ("kla_oracle.c", "kla_oracle_impl.h")
    )
    if force or src_newer or not os.path.exists(_LIB_PATH):
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def _ptr(x: Optional[np.ndarray]):
    return None if x is None else x.ctypes.data_as(ctypes.c_void_p)


def _prep(dtype, *arrays):
    return tuple(
        None if x is None else np.ascontiguousarray(np.asarray(x), dtype=dtype)
        for x in arrays
    )


def _suffix(dtype) -> str:
    dtype = np.dtype(dtype)
    if dtype == np.float64:
        return "f64"
    if dtype == np.float32:
        return "f32"
    raise TypeError(f"oracle supports float64/float32, got {dtype}")


class ScanOut(NamedTuple):
    y: np.ndarray
    y_var: np.ndarray
    lam: np.ndarray
    eta: np.ndarray


class ScanGrads(NamedTuple):
    dv: np.ndarray
    dlambda_v: np.ndarray
    dk: np.ndarray
    dq: np.ndarray
    da: np.ndarray
    dp: np.ndarray
    dlam0: np.ndarray
    deta0: np.ndarray


def scan_fwd(v, lambda_v, k, q, a, p, lam0=None, eta0=None, *, prior=False,
             floor_phi=False, dtype=np.float64) -> ScanOut:
    """Sequential forward scan; the reference's ``kla_scan_reference``
    (``kla_ops.py:334-362``). ``floor_phi=True`` reproduces ``kla_step``'s
    floor on phi (``kla_ops.py:310-312``); the default matches the reference's
    parallel torch path, which leaves phi unfloored (``kla_ops.py:238``)."""
    lib = _load()
    v, lambda_v, k, q, a, p, lam0, eta0 = _prep(dtype, v, lambda_v, k, q, a, p, lam0, eta0)
    B, L, M = v.shape
    S = k.shape[2]
    y = np.empty((B, L, M), dtype)
    y_var = np.empty((B, L, M), dtype)
    lam = np.empty((B, M, S), dtype)
    eta = np.empty((B, M, S), dtype)
    fn = getattr(lib, "kla_oracle_fwd_" + _suffix(dtype))
    fn.restype = ctypes.c_int
    rc = fn(ctypes.c_int64(B), ctypes.c_int64(L), ctypes.c_int64(M), ctypes.c_int64(S),
            _ptr(v), _ptr(lambda_v), _ptr(k), _ptr(q), _ptr(a), _ptr(p),
            _ptr(lam0), _ptr(eta0), ctypes.c_int(int(prior)), ctypes.c_int(int(floor_phi)),
            _ptr(y), _ptr(y_var), _ptr(lam), _ptr(eta))
    if rc != 0:
        raise ValueError(f"kla_oracle_fwd returned {rc}")
    return ScanOut(y, y_var, lam, eta)


def scan_bwd(v, lambda_v, k, q, a, p, dy, dyvar=None, lam0=None, eta0=None,
             dlam_fin=None, deta_fin=None, *, prior=False, floor_phi=False,
             dtype=np.float64) -> ScanGrads:
    """Exact adjoint of :func:`scan_fwd` for the loss
    ``sum(dy*y) + sum(dyvar*y_var) + sum(dlam_fin*lam) + sum(deta_fin*eta)``."""
    lib = _load()
    (v, lambda_v, k, q, a, p, dy, dyvar, lam0, eta0, dlam_fin, deta_fin) = _prep(
        dtype, v, lambda_v, k, q, a, p, dy, dyvar, lam0, eta0, dlam_fin, deta_fin)
    B, L, M = v.shape
    S = k.shape[2]
    out = ScanGrads(
        np.zeros((B, L, M), dtype), np.zeros((B, L, M), dtype),
        np.zeros((B, L, S), dtype), np.zeros((B, L, S), dtype),
        np.zeros((M, S), dtype), np.zeros((M, S), dtype),
        np.zeros((B, M, S), dtype), np.zeros((B, M, S), dtype))
    if L == 0:
        if dlam_fin is not None:
            out.dlam0[...] = dlam_fin
        if deta_fin is not None:
            out.deta0[...] = deta_fin
        return out
    fn = getattr(lib, "kla_oracle_bwd_" + _suffix(dtype))
    fn.restype = ctypes.c_int
    rc = fn(ctypes.c_int64(B), ctypes.c_int64(L), ctypes.c_int64(M), ctypes.c_int64(S),
            _ptr(v), _ptr(lambda_v), _ptr(k), _ptr(q), _ptr(a), _ptr(p),
            _ptr(lam0), _ptr(eta0), ctypes.c_int(int(prior)), ctypes.c_int(int(floor_phi)),
            _ptr(dy), _ptr(dyvar), _ptr(dlam_fin), _ptr(deta_fin),
            *[_ptr(x) for x in out])
    if rc != 0:
        raise ValueError(f"kla_oracle_bwd returned {rc}")
    return out


def step(v, lambda_v, k, q, a, p, lam, eta, *, prior=False, dtype=np.float64) -> ScanOut:
    """One decode step, ``kla_step`` (``kla_ops.py:293-331``). v, lambda_v: [B, M];
    k, q: [B, S]; lam, eta: [B, M, S]."""
    lib = _load()
    v, lambda_v, k, q, a, p, lam, eta = _prep(dtype, v, lambda_v, k, q, a, p, lam, eta)
    B, M = v.shape
    S = k.shape[1]
    y = np.empty((B, M), dtype)
    y_var = np.empty((B, M), dtype)
    lam_o = np.empty((B, M, S), dtype)
    eta_o = np.empty((B, M, S), dtype)
    fn = getattr(lib, "kla_oracle_step_" + _suffix(dtype))
    fn.restype = ctypes.c_int
    rc = fn(ctypes.c_int64(B), ctypes.c_int64(M), ctypes.c_int64(S),
            _ptr(v), _ptr(lambda_v), _ptr(k), _ptr(q), _ptr(a), _ptr(p),
            _ptr(lam), _ptr(eta), ctypes.c_int(int(prior)),
            _ptr(y), _ptr(y_var), _ptr(lam_o), _ptr(eta_o))
    if rc != 0:
        raise ValueError(f"kla_oracle_step returned {rc}")
    return ScanOut(y, y_var, lam_o, eta_o)
