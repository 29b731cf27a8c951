"""The CPU oracle against the golden vectors the reference package produced.

The golden files hold ``kla.ops.kla_scan_reference`` (float64) and its torch
autograd gradients (``tests/golden/make_golden.py``). The oracle must reproduce
them to float64 rounding before anything else is allowed to trust it.
"""

import numpy as np
import pytest

from conftest import golden_names, load_golden
from oracle import kla_oracle as O

RTOL = 1e-9
ATOL = 1e-11


def _close(got, ref, what):
    scale = np.abs(ref).max() + 1.0
    err = np.abs(got - ref).max() / scale
    assert np.isfinite(got).all(), f"{what}: non-finite"
    assert err < RTOL, f"{what}: {err:.2e}"


@pytest.mark.parametrize("name", golden_names())
def test_oracle_matches_reference_golden(name):
    g = load_golden(name)
    prior = bool(g["prior"])
    ins = [g[n] for n in ("v", "lambda_v", "k", "q", "a", "p")]
    lam0, eta0 = g.get("lam0"), g.get("eta0")
    # the sequential reference floors phi (kla_ops.py:310-312)
    f = O.scan_fwd(*ins, lam0, eta0, prior=prior, floor_phi=True)
    _close(f.y, g["y"], "y")
    _close(f.y_var, g["y_var"], "y_var")
    _close(f.lam, g["lam_fin"], "lam_fin")
    _close(f.eta, g["eta_fin"], "eta_fin")
    b = O.scan_bwd(*ins, g["dy"], g["dyvar"], lam0, eta0, g.get("dlam_fin"),
                   g.get("deta_fin"), prior=prior, floor_phi=True)
    for n in ("dv", "dlambda_v", "dk", "dq", "da", "dp"):
        _close(getattr(b, n), g[n], n)
    if lam0 is not None:
        _close(b.dlam0, g["dlam0"], "dlam0")
        _close(b.deta0, g["deta0"], "deta0")


@pytest.mark.parametrize("prior", [False, True])
def test_oracle_step_matches_reference_golden(prior):
    g = load_golden("step")
    tag = "_prior" if prior else ""
    s = O.step(g["v"], g["lambda_v"], g["k"], g["q"], g["a"], g["p"], g["lam"], g["eta"], prior=prior)
    _close(s.y, g["y" + tag], "y")
    _close(s.y_var, g["y_var" + tag], "y_var")
    _close(s.lam, g["lam_out" + tag], "lam")
    _close(s.eta, g["eta_out" + tag], "eta")


def test_unfloored_phi_differs_only_below_eps():
    """The default parallel path leaves phi unfloored (kla_ops.py:238); on
    well-conditioned inputs that equals the floored sequential reference."""
    g = load_golden("cfg2small")
    ins = [g[n] for n in ("v", "lambda_v", "k", "q", "a", "p")]
    f0 = O.scan_fwd(*ins, g["lam0"], g["eta0"], floor_phi=False)
    f1 = O.scan_fwd(*ins, g["lam0"], g["eta0"], floor_phi=True)
    assert np.abs(f0.y - f1.y).max() < 1e-10
    assert np.abs(f0.y_var - f1.y_var).max() < 1e-10


def test_oracle_split_equals_full():
    """State carry: scanning two halves equals one scan (tests/test_ops.py:63-75)."""
    g = load_golden("cfg2small")
    v, lv, k, q, a, p = [g[n] for n in ("v", "lambda_v", "k", "q", "a", "p")]
    full = O.scan_fwd(v, lv, k, q, a, p)
    mid = 77
    h = O.scan_fwd(v[:, :mid], lv[:, :mid], k[:, :mid], q[:, :mid], a, p)
    t = O.scan_fwd(v[:, mid:], lv[:, mid:], k[:, mid:], q[:, mid:], a, p, h.lam, h.eta)
    np.testing.assert_allclose(np.concatenate([h.y, t.y], 1), full.y, rtol=1e-12, atol=1e-13)
    np.testing.assert_allclose(t.lam, full.lam, rtol=1e-12)


def test_oracle_float32_close_to_float64():
    g = load_golden("backends")
    ins = [g[n] for n in ("v", "lambda_v", "k", "q", "a", "p")]
    f64 = O.scan_fwd(*ins)
    f32 = O.scan_fwd(*ins, dtype=np.float32)
    assert f32.y.dtype == np.float32
    np.testing.assert_allclose(f32.y, f64.y, rtol=1e-4, atol=1e-5)
