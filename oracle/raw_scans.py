"""CPU restatement (numpy, float64) of the reference's raw scan pair. TEST INFRASTRUCTURE
ONLY: imported by tests/, the smoke check and the benchmark's CPU leg, never by the product.

Follows src/kla/ops/kernels/triton/tiled_mobius_scan.py of the reference:
  * mobius_fwd   the recurrence the tiled kernel evaluates, lam_t = num/max(den, 1e-12)
                 (:98-102; the trace normalisation there cancels in num/den);
  * mobius_bwd   TiledMobiusScan.backward (:266-279);
  * affine_fwd   eta_t = alpha_t eta_{t-1} + r_t (:160-203);
  * affine_bwd   TiledAffineScan.backward (:289-296).
Pinned by tests/golden/raw_*.npz, which were produced with the reference's own CPU
functions (its trace-normalised Moebius combine under its sequential scan, and torch
autograd of the defining recurrences); see tests/golden/make_golden_raw.py.
"""

from __future__ import annotations

import numpy as np

EPS = 1e-12


def mobius_fwd(A, B, C, D, lam0=None):
    A, B, C, D = (np.asarray(x, dtype=np.float64) for x in (A, B, C, D))
    Bn, L, M, S = A.shape
    lam = np.ones((Bn, M, S)) if lam0 is None else np.asarray(lam0, dtype=np.float64).copy()
    out = np.empty_like(A)
    for t in range(L):
        lam = (A[:, t] * lam + B[:, t]) / np.maximum(C[:, t] * lam + D[:, t], EPS)
        out[:, t] = lam
    return out


def mobius_bwd(A, B, C, D, lam0, lam, dlam):
    A, B, C, D, lam, dlam = (np.asarray(x, dtype=np.float64) for x in (A, B, C, D, lam, dlam))
    Bn, L, M, S = A.shape
    lam0 = np.ones((Bn, M, S)) if lam0 is None else np.asarray(lam0, dtype=np.float64)
    lam_prev = np.concatenate([lam0[:, None], lam[:, :-1]], axis=1)
    den = np.maximum(C * lam_prev + D, EPS)
    gain = (A * D - B * C) / (den * den)
    nu = np.empty_like(A)
    carry = np.zeros((Bn, M, S))
    for t in range(L - 1, -1, -1):
        nu[:, t] = dlam[:, t] + carry
        carry = gain[:, t] * nu[:, t]
    nod = nu / den
    return nod * lam_prev, nod, -nod * lam * lam_prev, -nod * lam, carry


def affine_fwd(alpha, r):
    alpha, r = np.asarray(alpha, dtype=np.float64), np.asarray(r, dtype=np.float64)
    eta = np.zeros_like(alpha[:, 0])
    out = np.empty_like(alpha)
    for t in range(alpha.shape[1]):
        eta = alpha[:, t] * eta + r[:, t]
        out[:, t] = eta
    return out


def affine_bwd(alpha, eta, deta):
    alpha, eta, deta = (np.asarray(x, dtype=np.float64) for x in (alpha, eta, deta))
    eta_prev = np.concatenate([np.zeros_like(eta[:, :1]), eta[:, :-1]], axis=1)
    mu = np.empty_like(alpha)
    carry = np.zeros_like(alpha[:, 0])
    for t in range(alpha.shape[1] - 1, -1, -1):
        mu[:, t] = deta[:, t] + carry
        carry = alpha[:, t] * mu[:, t]
    return mu * eta_prev, mu
