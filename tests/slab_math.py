"""Plain numpy (float64) restatement of the slab aggregates used by the
sequence-sharded scan, written from the filter equations
(src/kla/ops/kla_ops.py:9-14, 293-331), not from the CUDA kernels. Test
infrastructure: the GPU tests compare the kernels' aggregates with these, the
CPU tests use them in place of the kernels."""

import numpy as np

EPS = 1e-12


def _coeffs(a, p):
    a2 = np.maximum(a * a, EPS)
    return a[None], a2[None], np.maximum(p, EPS)[None]


def forward_aggregate(v, lambda_v, k, a, p):
    """[B, M, S, 8]: the slab's map on (x, w, z), P = w/x, mean = z/x."""
    B, L, M = v.shape
    S = k.shape[2]
    a_, a2, p_ = _coeffs(a, p)
    m = np.zeros((B, M, S, 3, 3))
    m[..., 0, 0] = m[..., 1, 1] = m[..., 2, 2] = 1.0
    for t in range(L):
        phi = lambda_v[:, t, :, None] * k[:, t, None, :] ** 2
        r = (v[:, t] * lambda_v[:, t])[:, :, None] * k[:, t, None, :]
        T = np.zeros((B, M, S, 3, 3))
        T[..., 0, 0] = 1 + p_ * phi
        T[..., 0, 1] = a2 * phi
        T[..., 1, 0] = p_
        T[..., 1, 1] = a2
        T[..., 2, 0] = r * p_
        T[..., 2, 1] = r * a2
        T[..., 2, 2] = a_
        m = T @ m
        m = m / (m[..., 0:1, 0:1] + m[..., 0:1, 1:2])
    out = np.zeros((B, M, S, 8))
    out[..., 0], out[..., 1] = m[..., 0, 0], m[..., 0, 1]
    out[..., 2], out[..., 3] = m[..., 1, 0], m[..., 1, 1]
    out[..., 4], out[..., 5], out[..., 6] = m[..., 2, 0], m[..., 2, 1], m[..., 2, 2]
    return out


def adjoint_aggregate(v, lambda_v, k, q, a, p, dy, dyvar, lam0, eta0, prior=False):
    """[B, M, S, 8]: (K00 K01 K11 b0 b1 P_end mean_end 0)."""
    B, L, M = v.shape
    S = k.shape[2]
    a_, a2, p_ = _coeffs(a, p)
    P = 1.0 / lam0 if lam0 is not None else np.ones((B, M, S))
    mean = eta0 * P if eta0 is not None else np.zeros((B, M, S))
    K00, K01, K11 = np.ones((B, M, S)), np.zeros((B, M, S)), np.ones((B, M, S))
    b0, b1 = np.zeros((B, M, S)), np.zeros((B, M, S))
    if dyvar is None:
        dyvar = np.zeros_like(dy)
    for t in range(L):
        kk, qq = k[:, t, None, :], q[:, t, None, :]
        phi = lambda_v[:, t, :, None] * kk ** 2
        r = (v[:, t] * lambda_v[:, t])[:, :, None] * kk
        Pp = a2 * P + p_
        g = 1.0 / (1.0 + phi * Pp)
        P = Pp * g
        mean = g * (a_ * mean + Pp * r)
        j00, j01, j11 = a2 * g * g, a2 * g * (r - phi * mean), a_ * g
        e0, e1 = dyvar[:, t, :, None] * qq ** 2, dy[:, t, :, None] * qq
        if prior:
            e0, e1 = e0 * a2, e1 * a_
        K00, K01, K11 = K00 * j00, K00 * j01 + K01 * j11, K11 * j11
        b0 = b0 + K00 * e0 + K01 * e1
        b1 = b1 + K11 * e1
    out = np.zeros((B, M, S, 8))
    for i, x in enumerate((K00, K01, K11, b0, b1, P, mean)):
        out[..., i] = x
    return out
