"""Raw scan pair (Moebius / affine scans over materialised coefficients): the numpy oracle
against the golden vectors made with the reference's CPU code, and the B200 kernels against
the oracle through the C ABI."""

import glob
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

from oracle import raw_scans  # noqa: E402

CASES = sorted(os.path.basename(p)[4:-4] for p in glob.glob(os.path.join(HERE, "golden", "raw_*.npz")))
RTOL, ATOL = 1e-5, 1e-6  # float32 bar of the hot path


def load(name):
    return dict(np.load(os.path.join(HERE, "golden", f"raw_{name}.npz")))


def test_cases_present():
    assert CASES == ["noprior", "odd", "small", "wide"]


@pytest.mark.parametrize("name", CASES)
def test_oracle_matches_golden(name):
    g = load(name)
    lam0 = g.get("lam0")
    lam = raw_scans.mobius_fwd(g["A"], g["B"], g["C"], g["D"], lam0)
    np.testing.assert_allclose(lam, g["lam"], rtol=1e-11, atol=1e-13)
    dA, dB, dC, dD, dlam0 = raw_scans.mobius_bwd(g["A"], g["B"], g["C"], g["D"], lam0, lam, g["dlam"])
    for got, key in ((dA, "dA"), (dB, "dB"), (dC, "dC"), (dD, "dD")):
        np.testing.assert_allclose(got, g[key], rtol=1e-9, atol=1e-11, err_msg=key)
    if lam0 is not None:
        np.testing.assert_allclose(dlam0, g["dlam0"], rtol=1e-9, atol=1e-11)
    eta = raw_scans.affine_fwd(g["alpha"], g["r"])
    np.testing.assert_allclose(eta, g["eta"], rtol=1e-11, atol=1e-13)
    dal, dr = raw_scans.affine_bwd(g["alpha"], eta, g["deta"])
    np.testing.assert_allclose(dal, g["dalpha"], rtol=1e-9, atol=1e-11)
    np.testing.assert_allclose(dr, g["dr"], rtol=1e-9, atol=1e-11)


def test_cpu_tensors_are_refused():
    torch = pytest.importorskip("torch")
    import kla_b200
    from importlib import import_module

    rs = import_module("kalman-linear-attention_b200.rawscan")
    x = torch.ones(1, 4, 2, 2)
    with pytest.raises(NotImplementedError, match="CUDA"):
        rs.mobius_scan_b200(x, x, x, x)
    with pytest.raises(NotImplementedError, match="CUDA"):
        rs.affine_scan_b200(x, x)
    assert kla_b200.mobius_scan_b200 is rs.mobius_scan_b200


# ----------------------------------------------------------------------- GPU

def _t(a, dev, grad=False):
    import torch

    return torch.tensor(np.asarray(a, dtype=np.float32), device=dev, requires_grad=grad)


def _close(got, ref, what):
    got = got.detach().double().cpu().numpy()
    err = np.abs(got - ref) / (ATOL + RTOL * np.abs(ref))
    assert err.max() <= 1.0, f"{what}: worst elementwise error {err.max():.2f} x the float32 tolerance"


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_kernels_match_golden(name):
    import torch
    import kla_b200

    dev = torch.device("cuda:0")
    g = load(name)
    A, B, C, D = (_t(g[k], dev, True) for k in "ABCD")
    lam0 = _t(g["lam0"], dev, True) if "lam0" in g else None
    lam = kla_b200.mobius_scan_b200(A, B, C, D, lam0)
    # the float32 inputs are roundings of the float64 ones: compare with the oracle on the rounded inputs
    f32 = {k: np.asarray(g[k], dtype=np.float32).astype(np.float64) for k in ("A", "B", "C", "D", "dlam", "alpha", "r", "deta")}
    l0 = np.asarray(g["lam0"], dtype=np.float32).astype(np.float64) if "lam0" in g else None
    ref_lam = raw_scans.mobius_fwd(f32["A"], f32["B"], f32["C"], f32["D"], l0)
    _close(lam, ref_lam, "lam")
    lam.backward(_t(g["dlam"], dev))
    ref = raw_scans.mobius_bwd(f32["A"], f32["B"], f32["C"], f32["D"], l0, ref_lam, f32["dlam"])
    for t, r, what in zip((A, B, C, D), ref, ("dA", "dB", "dC", "dD")):
        _close(t.grad, r, what)
    if lam0 is not None:
        _close(lam0.grad, ref[4], "dlam0")

    alpha, r = _t(g["alpha"], dev, True), _t(g["r"], dev, True)
    eta = kla_b200.affine_scan_b200(alpha, r)
    ref_eta = raw_scans.affine_fwd(f32["alpha"], f32["r"])
    _close(eta, ref_eta, "eta")
    eta.backward(_t(g["deta"], dev))
    ref_da, ref_dr = raw_scans.affine_bwd(f32["alpha"], ref_eta, f32["deta"])
    _close(alpha.grad, ref_da, "dalpha")
    _close(r.grad, ref_dr, "dr")
    L = __import__("importlib").import_module("kalman-linear-attention_b200._lib")
    assert L.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(1, 1, 1, 1), (2, 8, 4, 8), (1, 17, 33, 4), (3, 100, 7, 16), (1, 64, 64, 16)])
def test_kernels_match_oracle_on_seeded_inputs(shape):
    import torch
    import kla_b200

    dev = torch.device("cuda:0")
    Bn, L, M, S = shape
    rng = np.random.default_rng(sum(shape))
    # a contracting map (gain < 1), like the filter's own leaves: float32 rounding is not amplified along the scan
    A = (0.5 + 0.5 * rng.random(shape)).astype(np.float32)
    Bc = (0.1 * rng.random(shape)).astype(np.float32)
    C = (0.2 * rng.random(shape)).astype(np.float32)
    D = np.ones(shape, dtype=np.float32)
    lam0 = (0.5 + rng.random((Bn, M, S))).astype(np.float32)
    dl = rng.standard_normal(shape).astype(np.float32)
    tA, tB, tC, tD = (_t(x, dev, True) for x in (A, Bc, C, D))
    t0 = _t(lam0, dev, True)
    lam = kla_b200.mobius_scan_b200(tA, tB, tC, tD, t0)
    ref_lam = raw_scans.mobius_fwd(A, Bc, C, D, lam0)
    _close(lam, ref_lam, "lam")
    lam.backward(_t(dl, dev))
    ref = raw_scans.mobius_bwd(A, Bc, C, D, lam0, ref_lam, dl)
    for t, r, what in zip((tA, tB, tC, tD, t0), ref, ("dA", "dB", "dC", "dD", "dlam0")):
        _close(t.grad, r, what)
    al = (0.5 + 0.5 * rng.random(shape)).astype(np.float32)
    rr = rng.standard_normal(shape).astype(np.float32)
    tal, trr = _t(al, dev, True), _t(rr, dev, True)
    eta = kla_b200.affine_scan_b200(tal, trr)
    ref_eta = raw_scans.affine_fwd(al, rr)
    _close(eta, ref_eta, "eta")
    eta.backward(_t(dl, dev))
    rda, rdr = raw_scans.affine_bwd(al, ref_eta, dl)
    _close(tal.grad, rda, "dalpha")
    _close(trr.grad, rdr, "dr")


@pytest.mark.gpu
def test_full_size_properties():
    """At the benchmark's size the oracle is too slow, so check properties that do not depend
    on size: alpha = 1 turns the affine scan into a running sum; C = 0, D = 1 turns the Moebius
    scan into the affine scan; one lane block equals the same block scanned on its own."""
    import torch
    import kla_b200

    dev = torch.device("cuda:0")
    Bn, L, M, S = 2, 4096, 256, 16
    g = torch.Generator(device="cpu").manual_seed(0)
    r = torch.randn(Bn, L, M, S, generator=g).to(dev)
    ones = torch.ones_like(r)
    eta = kla_b200.affine_scan_b200(ones, r)
    ref = torch.cumsum(r.double(), dim=1)
    assert torch.allclose(eta.double(), ref, rtol=1e-4, atol=1e-3)
    alpha = (0.5 + 0.5 * torch.rand(Bn, L, M, S, generator=g)).to(dev)
    eta = kla_b200.affine_scan_b200(alpha, r)
    lam = kla_b200.mobius_scan_b200(alpha, r, torch.zeros_like(r), ones, torch.zeros(Bn, M, S, device=dev))
    assert torch.equal(lam, eta) or torch.allclose(lam, eta, rtol=1e-6, atol=1e-6)
    blk = kla_b200.affine_scan_b200(alpha[:, :, 64:96].contiguous(), r[:, :, 64:96].contiguous())
    assert torch.equal(blk, eta[:, :, 64:96])
