"""Generate the golden vectors under tests/golden/ from the reference package.

Run once, in a container where the reference tree is importable:

    PYTHONPATH=<reference>/src python tests/golden/make_golden.py

Every case stores its inputs and the reference's own outputs: the float64
sequential scan ``kla.ops.kla_scan_reference`` (the reference's correctness
anchor) differentiated with torch autograd, plus -- for the noise-floor report
-- the reference's float32 ``backend="torch"`` results on the same inputs.
Inputs follow the reference's own seeded generators:

* ``backends``  tests/test_backends.py:136-150 (``make_inputs``, seed 0)
* ``cfg2small`` the coefficient distributions of the headline raw-op workload
  (a = sigmoid(N), p = softplus(N), lambda_v = 1/softplus(N), l2-normalised
  k, q) at a size that runs in seconds
* ``gradcheck`` the shape of tests/test_gradcheck.py:35-57
* edge cases    tests/test_backends.py:421-564 and tests/test_blocks.py:164-179
* ``step``      one ``kla_step`` call (src/kla/ops/kla_ops.py:293-331)
"""

import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

from kla.ops import KLAState, kla_scan, kla_scan_reference, kla_step

HERE = os.path.dirname(os.path.abspath(__file__))
F64 = torch.float64


def backends_inputs(B=2, L=64, M=16, S=8):
    g = torch.Generator(device="cpu").manual_seed(0)
    return [
        torch.randn(B, L, M, generator=g),
        torch.rand(B, L, M, generator=g) + 0.5,
        torch.randn(B, L, S, generator=g) * 0.3,
        torch.randn(B, L, S, generator=g) * 0.3,
        torch.rand(M, S, generator=g) * 0.5 + 0.4,
        torch.rand(M, S, generator=g) * 0.05 + 0.01,
    ]


def cfg2_inputs(B, L, M, S, normalise=True):
    g = torch.Generator(device="cpu").manual_seed(0)
    v = torch.randn(B, L, M, generator=g)
    lambda_v = 1.0 / F.softplus(torch.randn(B, L, M, generator=g))
    k = torch.randn(B, L, S, generator=g)
    q = torch.randn(B, L, S, generator=g)
    if normalise:
        k = k / k.norm(dim=-1, keepdim=True)
        q = q / q.norm(dim=-1, keepdim=True)
    a = torch.sigmoid(torch.randn(M, S, generator=g))
    p = F.softplus(torch.randn(M, S, generator=g))
    return [v, lambda_v, k, q, a, p]


def run_case(name, inputs, *, state=False, prior=False, loss="rand", fp32=True):
    """Reference forward + autograd in float64 (and float32 through the torch backend)."""
    ins = [t.to(F64).detach().clone().requires_grad_(True) for t in inputs]
    B, L, M = ins[0].shape
    S = ins[2].shape[2]
    g = torch.Generator(device="cpu").manual_seed(1)
    out = {n: t.detach().numpy() for n, t in zip(("v", "lambda_v", "k", "q", "a", "p"), ins)}
    out["prior"] = np.array(int(prior))
    if loss == "rand":
        dy = torch.randn(B, L, M, generator=g, dtype=F64)
        dyvar = torch.randn(B, L, M, generator=g, dtype=F64)
    init = None
    extra = []
    if state:
        lam0 = (torch.rand(B, M, S, generator=g, dtype=F64) * 2 + 0.5).requires_grad_(True)
        eta0 = torch.randn(B, M, S, generator=g, dtype=F64).requires_grad_(True)
        dlam = torch.randn(B, M, S, generator=g, dtype=F64)
        deta = torch.randn(B, M, S, generator=g, dtype=F64)
        init = KLAState(lam0, eta0)
        extra = [lam0, eta0]
        out.update(lam0=lam0.detach().numpy(), eta0=eta0.detach().numpy(),
                   dlam_fin=dlam.numpy(), deta_fin=deta.numpy())
    y, y_var, st = kla_scan_reference(*ins, initial_state=init, decode_from_prior=prior)
    if loss == "rand":
        total = (y * dy).sum() + (y_var * dyvar).sum()
    else:  # the loss of tests/test_backends.py:307
        total = y.square().sum() + y_var.sum()
        dy, dyvar = (2 * y).detach(), torch.ones_like(y_var)
    if state:
        total = total + (st.lam * dlam).sum() + (st.eta * deta).sum()
    grads = torch.autograd.grad(total, ins + extra)
    out.update(dy=dy.numpy(), dyvar=dyvar.numpy(), y=y.detach().numpy(),
               y_var=y_var.detach().numpy(), lam_fin=st.lam.detach().numpy(),
               eta_fin=st.eta.detach().numpy())
    names = ["dv", "dlambda_v", "dk", "dq", "da", "dp"] + (["dlam0", "deta0"] if state else [])
    out.update({n: t.numpy() for n, t in zip(names, grads)})
    if fp32:
        # the reference's float32 CPU path on the same inputs (noise-floor report)
        ins32 = [t.detach().float().requires_grad_(True) for t in ins]
        init32 = None
        ex32 = []
        if state:
            l32 = lam0.detach().float().requires_grad_(True)
            e32 = eta0.detach().float().requires_grad_(True)
            init32, ex32 = KLAState(l32, e32), [l32, e32]
        y32, yv32, st32 = kla_scan(*ins32, initial_state=init32, backend="torch",
                                   scan_impl="doubling", decode_from_prior=prior)
        tot32 = (y32 * dy.float()).sum() + (yv32 * dyvar.float()).sum()
        if state:
            tot32 = tot32 + (st32.lam * dlam.float()).sum() + (st32.eta * deta.float()).sum()
        g32 = torch.autograd.grad(tot32, ins32 + ex32)
        out.update(ref32_y=y32.detach().numpy(), ref32_y_var=yv32.detach().numpy())
        out.update({"ref32_" + n: t.numpy() for n, t in zip(names, g32)})
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print(f"{name}: B,L,M,S={B},{L},{M},{S} state={state} prior={prior}")


def main():
    torch.set_num_threads(4)
    run_case("backends", backends_inputs(), loss="square")
    run_case("backends_state_prior", backends_inputs(L=37), state=True, prior=True)
    run_case("cfg2small", cfg2_inputs(2, 160, 24, 16), state=True)
    run_case("cfg2small_raw_kq", cfg2_inputs(1, 96, 8, 16, normalise=False))
    run_case("cfg2_long", cfg2_inputs(1, 2048, 4, 16), fp32=True)
    g = torch.Generator().manual_seed(0)
    run_case("gradcheck_shape", [
        torch.randn(1, 8, 3, generator=g, dtype=F64), torch.rand(1, 8, 3, generator=g, dtype=F64) + 0.5,
        torch.randn(1, 8, 2, generator=g, dtype=F64), torch.randn(1, 8, 2, generator=g, dtype=F64),
        torch.rand(3, 2, generator=g, dtype=F64) * 0.5 + 0.4, torch.rand(3, 2, generator=g, dtype=F64) * 0.05 + 0.01,
    ], state=True)
    # geometry cases: S, M that divide nothing (tests/test_backends.py:733-734)
    for S, M in ((1, 1), (3, 33), (17, 5), (33, 2), (64, 3)):
        run_case(f"geom_S{S}_M{M}", backends_inputs(B=2, L=19, M=M, S=S), state=True, fp32=False)
    # edge cases
    v, lv, k, q, a, p = backends_inputs()
    run_case("edge_p_zero", [v, lv, k, q, a, torch.zeros_like(p)], fp32=False)
    run_case("edge_p_negative", [v, lv, k, q, a, torch.full_like(p, -0.05)], fp32=False)
    run_case("edge_a_tiny", [v, lv, k, q, torch.full_like(a, 1e-10), p], fp32=False)
    run_case("edge_high_phi", [v, lv * 1e4, k, q, a, p], fp32=False)
    run_case("edge_zero_keys", [v, lv, torch.zeros_like(k), q, a, p], fp32=False)
    # one decode step (kla_step floors phi; so does kla_scan_reference)
    v, lv, k, q, a, p = [t.to(F64) for t in cfg2_inputs(3, 1, 20, 16)]
    g = torch.Generator().manual_seed(2)
    lam = torch.rand(3, 20, 16, generator=g, dtype=F64) * 3 + 0.2
    eta = torch.randn(3, 20, 16, generator=g, dtype=F64)
    res = {}
    for prior in (False, True):
        y, yv, st = kla_step(v[:, 0], lv[:, 0], k[:, 0], q[:, 0], a, p, KLAState(lam, eta),
                             decode_from_prior=prior)
        tag = "_prior" if prior else ""
        res.update({"y" + tag: y.numpy(), "y_var" + tag: yv.numpy(),
                    "lam_out" + tag: st.lam.numpy(), "eta_out" + tag: st.eta.numpy()})
    np.savez_compressed(os.path.join(HERE, "step.npz"), v=v[:, 0].numpy(), lambda_v=lv[:, 0].numpy(),
                        k=k[:, 0].numpy(), q=q[:, 0].numpy(), a=a.numpy(), p=p.numpy(),
                        lam=lam.numpy(), eta=eta.numpy(), **res)
    print("step")


if __name__ == "__main__":
    sys.exit(main())
