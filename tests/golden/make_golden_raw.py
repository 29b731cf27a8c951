"""Generate tests/golden/raw_*.npz: golden vectors for the raw scan pair.

    PYTHONPATH=<reference>/src python tests/golden/make_golden_raw.py

The reference's tiled scans themselves need Triton and a GPU, so the vectors come
from the reference's CPU code for the same maps, in float64:

* forward Moebius: the reference's trace-normalised combine
  (kla.ops.kla_ops._mobius_combine_tracenorm) under its sequential scan
  (kla.ops.scan.sequential_scan), folded onto lam0 as kla_scan_torch does
  (src/kla/ops/kla_ops.py:248-250);
* forward affine: kla.ops.kla_ops._affine_combine under the same scan (:279-280);
* gradients: torch autograd of those two computations, for a random upstream gradient.

Coefficients are built the way kla_scan_torch builds its leaves (:244-247, :275-277) from
the distributions of the headline workload, so they sit in the operating range.
"""

import os

import numpy as np
import torch
import torch.nn.functional as F

from kla.ops.kla_ops import _affine_combine, _mobius_combine_tracenorm
from kla.ops.scan import sequential_scan

HERE = os.path.dirname(os.path.abspath(__file__))
F64 = torch.float64


def leaves(B, L, M, S, seed):
    g = torch.Generator().manual_seed(seed)
    lam_v = 1.0 / F.softplus(torch.randn(B, L, M, generator=g, dtype=F64))
    k = F.normalize(torch.randn(B, L, S, generator=g, dtype=F64), dim=-1)
    v = torch.randn(B, L, M, generator=g, dtype=F64)
    a = torch.sigmoid(torch.randn(M, S, generator=g, dtype=F64))
    p = F.softplus(torch.randn(M, S, generator=g, dtype=F64))
    phi = lam_v[..., None] * (k * k)[:, :, None, :]
    r = (v * lam_v)[..., None] * k[:, :, None, :]
    a2 = a * a
    A = ((1.0 + p * phi) / a2).contiguous()
    Bc = phi.contiguous()
    C = (p / a2).expand_as(phi).contiguous()
    D = torch.ones_like(phi)
    lam0 = torch.rand(B, M, S, generator=g, dtype=F64) + 0.5
    dlam = torch.randn(B, L, M, S, generator=g, dtype=F64)
    return A, Bc, C, D, lam0, r, a, p, dlam


def case(name, B, L, M, S, seed, with_lam0):
    A, Bc, C, D, lam0, r, a, p, dout = leaves(B, L, M, S, seed)
    ins = [t.clone().requires_grad_(True) for t in (A, Bc, C, D)]
    l0 = lam0.clone().requires_grad_(True) if with_lam0 else None
    l0_ = (l0 if with_lam0 else torch.ones(B, M, S, dtype=F64)).unsqueeze(1)
    pA, pB, pC, pD = sequential_scan(_mobius_combine_tracenorm, tuple(ins), dim=1)
    lam = (pA * l0_ + pB) / (pC * l0_ + pD).clamp_min(1e-12)
    grads = torch.autograd.grad(lam, ins + ([l0] if with_lam0 else []), dout)
    out = dict(A=A, B=Bc, C=C, D=D, dlam=dout, lam=lam.detach(),
               dA=grads[0], dB=grads[1], dC=grads[2], dD=grads[3])
    if with_lam0:
        out.update(lam0=lam0, dlam0=grads[4])
    # affine leg: alpha_t = a / (a^2 + p lam_{t-1}) as in kla_scan_torch, r as above
    lam_prev = torch.cat([l0_.detach().expand(B, 1, M, S), lam.detach()[:, :-1]], dim=1)
    alpha = (a / (a * a + p * lam_prev)).clone().requires_grad_(True)
    rr = r.clone().requires_grad_(True)
    _, eta = sequential_scan(_affine_combine, (alpha, rr), dim=1)
    dal, dr = torch.autograd.grad(eta, (alpha, rr), dout)
    out.update(alpha=alpha.detach(), r=r, eta=eta.detach(), deta=dout, dalpha=dal, dr=dr)
    np.savez_compressed(os.path.join(HERE, f"raw_{name}.npz"), **{k_: v_.numpy() for k_, v_ in out.items()})
    print(name, {k_: tuple(v_.shape) for k_, v_ in out.items() if k_ in ("A", "lam0")})


if __name__ == "__main__":
    case("small", 2, 37, 5, 4, 0, True)         # N = 20: ragged tiles, N not a multiple of the CTA width
    case("noprior", 1, 32, 4, 16, 1, False)     # unit prior, whole tiles
    case("odd", 2, 9, 3, 3, 2, True)            # N = 9: not a multiple of 4 -> no TMA
    case("wide", 1, 10, 20, 16, 3, True)        # N = 320: three CTAs per row, the last one partial
