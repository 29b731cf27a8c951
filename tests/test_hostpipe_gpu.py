"""scan_fwd_bwd_host (batch chunks pipelined over several streams, host buffers in and out)
must give what one kla_scan_b200 + autograd call over the whole batch gives."""

import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import kla_b200  # noqa: E402


def _host(B, L, M, S, seed):
    g = torch.Generator().manual_seed(seed)
    F = torch.nn.functional
    h = dict(
        v=torch.randn(B, L, M, generator=g),
        lambda_v=1.0 / F.softplus(torch.randn(B, L, M, generator=g)),
        k=F.normalize(torch.randn(B, L, S, generator=g), dim=-1),
        q=F.normalize(torch.randn(B, L, S, generator=g), dim=-1),
        a=torch.sigmoid(torch.randn(M, S, generator=g)),
        p=F.softplus(torch.randn(M, S, generator=g)),
        dy=torch.randn(B, L, M, generator=g),
        dyvar=torch.randn(B, L, M, generator=g),
    )
    return {n: t.pin_memory() for n, t in h.items()}


def test_pageable_or_device_tensors_are_refused():
    h = {n: torch.zeros(1, 2, 2) for n in ("v", "lambda_v", "k", "q", "dy", "dyvar")}
    h.update(a=torch.zeros(2, 2), p=torch.zeros(2, 2))
    with pytest.raises(ValueError, match="pinned"):
        kla_b200.scan_fwd_bwd_host(h, "cuda:0")


@pytest.mark.gpu
@pytest.mark.parametrize("chunk,n_streams", [(1, 4), (2, 2), (3, 1), (8, 4)])
def test_host_pipeline_matches_one_shot(chunk, n_streams):
    dev = torch.device("cuda:0")
    B, L, M, S = 5, 70, 40, 16
    h = _host(B, L, M, S, 3)
    out = kla_b200.scan_fwd_bwd_host(h, dev, chunk=chunk, n_streams=n_streams)
    torch.cuda.synchronize()
    ins = [h[n].to(dev).requires_grad_(True) for n in ("v", "lambda_v", "k", "q", "a", "p")]
    y, y_var, _ = kla_b200.kla_scan_b200(*ins)
    grads = torch.autograd.grad([y, y_var], ins, [h["dy"].to(dev), h["dyvar"].to(dev)])
    ref = dict(y=y, y_var=y_var, dv=grads[0], dlambda_v=grads[1], dk=grads[2], dq=grads[3], da=grads[4], dp=grads[5])
    for name in ("y", "y_var", "dv", "dlambda_v"):
        assert torch.equal(out[name], ref[name].detach().cpu()), name          # same lanes, same kernels
    for name in ("dk", "dq"):                                                  # atomics: order of the channel sums varies
        torch.testing.assert_close(out[name], ref[name].cpu(), rtol=1e-5, atol=1e-5)
    for name in ("da", "dp"):                                                  # batch sum taken in a different order
        torch.testing.assert_close(out[name], ref[name].cpu(), rtol=1e-4, atol=1e-4)
    out2 = kla_b200.scan_fwd_bwd_host(h, dev, out=out, chunk=chunk, n_streams=n_streams)  # buffers are reused
    torch.cuda.synchronize()
    assert out2 is out and torch.equal(out["y"], ref["y"].detach().cpu())
