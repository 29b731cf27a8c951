"""The time-parallel form of the scan on one GPU (``time_chunks``): the sequence is cut into chunks that run side
by side from exact start states. Checked against the float64 oracle, not only against the lane-serial kernels."""

import importlib

import numpy as np
import pytest
import torch

from oracle import kla_oracle as O
from test_scan_gpu import INPUTS, REDUCED_SLACK, _oracle, _seeded, ratio, rel_err

pytestmark = pytest.mark.gpu
ops = importlib.import_module("kalman-linear-attention_b200.ops")


def _run(kb, g, chunks, *, prior=False, state=True, dtype=torch.float32):
    dev = "cuda"
    ins = [torch.tensor(g[n], dtype=torch.float32, device=dev) for n in INPUTS]
    ins = [t.to(dtype) if n in ("v", "lambda_v", "k", "q") else t for n, t in zip(INPUTS, ins)]
    ins = [t.requires_grad_(True) for t in ins]
    init, extra = None, []
    if state:
        lam0 = torch.tensor(g["lam0"], dtype=torch.float32, device=dev, requires_grad=True)
        eta0 = torch.tensor(g["eta0"], dtype=torch.float32, device=dev, requires_grad=True)
        init, extra = kb.KLAState(lam0, eta0), [lam0, eta0]
    y, y_var, st = kb.kla_scan_b200(*ins, initial_state=init, decode_from_prior=prior, time_chunks=chunks)
    f32 = lambda n: torch.tensor(g[n], dtype=torch.float32, device=dev)
    loss = (y * f32("dy")).sum() + (y_var * f32("dyvar")).sum()
    if state:
        loss = loss + (st.lam * f32("dlam_fin")).sum() + (st.eta * f32("deta_fin")).sum()
    return y, y_var, st, torch.autograd.grad(loss, ins + extra)


@pytest.fixture(scope="module")
def kb():
    import kla_b200

    return kla_b200


@pytest.mark.parametrize("chunks", [2, 4, 8])
@pytest.mark.parametrize("prior", [False, True])
def test_time_chunks_match_the_oracle(kb, chunks, prior):
    g = _seeded(2, 512, 24, 16, seed=21)
    f, b = _oracle(g, prior=prior)
    launches0 = ops._lib.load().kla_b200_launch_count()
    y, y_var, st, grads = _run(kb, g, chunks, prior=prior)
    torch.cuda.synchronize()
    assert ops._lib.load().kla_b200_launch_count() - launches0 == 6  # aggregate, fold, scan; the same three backwards
    names = ["dv", "dlambda_v", "dk", "dq", "da", "dp", "dlam0", "deta0"]
    rows = {"y": ratio(y, f.y), "y_var": ratio(y_var, f.y_var), "lam_fin": ratio(st.lam, f.lam), "eta_fin": ratio(st.eta, f.eta)}
    rows.update({n: ratio(gr, ref) for n, gr, ref in zip(names, grads, b)})
    print(f"\n  C={chunks} prior={prior}: " + " ".join(f"{n}={r:.2f}" for n, r in rows.items()))
    for n, r in rows.items():
        # the chunk start states pass through one float32 rounding of an exactly folded state, so the elementwise
        # budget is that of the plain kernels; the four reduced gradients keep theirs
        assert r <= (REDUCED_SLACK if n in ("dk", "dq", "da", "dp") else 2.0), (n, r)
    for n, gr, ref in zip(names, grads, b):
        assert rel_err(gr, ref) < 2e-3, (n, rel_err(gr, ref))


def test_time_chunks_agree_with_the_plain_kernels_bf16_and_no_state(kb):
    g = _seeded(3, 384, 40, 16, seed=22, state=False)
    for n in ("v", "lambda_v", "k", "q"):
        g[n] = torch.tensor(g[n]).to(torch.bfloat16).double().numpy()
    y1, yv1, st1, g1 = _run(kb, g, 1, state=False, dtype=torch.bfloat16)
    y4, yv4, st4, g4 = _run(kb, g, 3, state=False, dtype=torch.bfloat16)
    torch.testing.assert_close(y4, y1, rtol=2e-5, atol=2e-6)
    torch.testing.assert_close(yv4, yv1, rtol=2e-5, atol=2e-6)
    torch.testing.assert_close(st4.lam, st1.lam, rtol=2e-5, atol=2e-6)
    torch.testing.assert_close(st4.eta, st1.eta, rtol=2e-5, atol=2e-6)
    for a_, b_, n in zip(g4, g1, INPUTS):
        assert rel_err(a_.float(), b_.double().cpu().numpy()) < (1e-2 if a_.dtype == torch.bfloat16 else 1e-4), n


def test_long_sequence_in_chunks_against_oracle(kb):
    """B=1, T=32768 in 8 chunks of 4096: the aggregates are products of 4096 step maps, rescaled as they go.
    State, y and all gradients against the float64 oracle."""
    g = _seeded(1, 32768, 32, 16, seed=23)
    f, b = _oracle(g)
    ins = [g[n] for n in INPUTS]
    b32 = O.scan_bwd(*ins, g["dy"], g["dyvar"], g["lam0"], g["eta0"], g["dlam_fin"], g["deta_fin"], dtype=np.float32)
    y, y_var, st, grads = _run(kb, g, 8)
    _, _, _, grads1 = _run(kb, g, 1)
    names = ["dv", "dlambda_v", "dk", "dq", "da", "dp", "dlam0", "deta0"]
    rows = {"y": ratio(y, f.y), "y_var": ratio(y_var, f.y_var), "lam_fin": ratio(st.lam, f.lam), "eta_fin": ratio(st.eta, f.eta)}
    rows.update({n: ratio(gr, ref) for n, gr, ref in zip(names, grads, b)})
    print("\n  T=32768, |err|/(1e-6 + 1e-5|ref|) against the float64 oracle: 8 chunks / plain kernels / float32 oracle")
    for i, n in enumerate(names):
        print(f"    {n:10s} {rows[n]:8.2f} {ratio(grads1[i], b[i]):8.2f} {ratio(b32[i], b[i]):8.2f}")
    for n, r in rows.items():
        if n in ("da", "dp"):
            # sums over 32768 steps: float32 summation noise grows with the length of the sum; the bound is the
            # reference's own gradient contract (tests/test_backends.py:54) and the noise of the plain kernels
            i = names.index(n)
            assert rel_err(grads[i], b[i]) < 2e-3 and r <= max(REDUCED_SLACK, 2.0 * ratio(grads1[i], b[i])), (n, r)
        else:
            assert r <= (REDUCED_SLACK if n in ("dk", "dq") else 2.0), (n, r)


def test_views_that_cannot_be_chunked_fall_back(kb):
    g = _seeded(2, 256, 16, 16, seed=24, state=False)
    dev = "cuda"
    wide = torch.zeros(2, 300, 16, device=dev)
    wide[:, :256] = torch.tensor(g["v"], dtype=torch.float32, device=dev)
    v = wide[:, :256]  # batch stride 300 rows: not L x the time stride
    rest = [torch.tensor(g[n], dtype=torch.float32, device=dev) for n in INPUTS[1:]]
    with torch.no_grad():
        y4, _, _ = kb.kla_scan_b200(v, *rest, time_chunks=4)
        y1, _, _ = kb.kla_scan_b200(v.contiguous(), *rest, time_chunks=1)
    assert torch.equal(y4, y1)
