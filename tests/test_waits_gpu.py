"""A bounded wait inside a kernel that runs out: the kernel must return, the device status must say where, and
the next ordinary launch on the same device must be correct.

Every hand-over between the warps of a scan kernel is a bounded wait on a shared-memory barrier. Nothing in
normal operation makes one run out, so this test makes it: ``kla_b200_test_hooks`` shortens the limit to a few
milliseconds and tells the loader warp to leave the hand-over of one tile incomplete. The tile's data is loaded
all the same; no kernel faults, traps or waits without a bound.
"""

import importlib

import pytest
import torch

pytestmark = pytest.mark.gpu

L = importlib.import_module("kalman-linear-attention_b200._lib")


def _inputs(requires_grad):
    g = torch.Generator().manual_seed(3)
    B, T, M, S = 2, 96, 48, 16
    v = torch.randn(B, T, M, generator=g)
    lv = 0.5 + torch.rand(B, T, M, generator=g)
    k, q = 0.3 * torch.randn(B, T, S, generator=g), 0.3 * torch.randn(B, T, S, generator=g)
    a, p = 0.4 + 0.5 * torch.rand(M, S, generator=g), 0.01 + 0.05 * torch.rand(M, S, generator=g)
    return [t.cuda().requires_grad_(requires_grad) for t in (v, lv, k, q, a, p)]


@pytest.fixture
def hooks():
    lib = L.load()
    yield lib
    assert lib.kla_b200_test_hooks(0, -1) == 0  # back to one second, nothing skipped


# With segments forced, every sequence is handed from CTA to CTA; a CTA stalled on the incomplete tile keeps the
# one after it waiting for the hand-over, and that bounded wait (site 9 forward, 19 backward) may be the first to
# run out.
@pytest.mark.parametrize("segments", [None, 3])
def test_forward_wait_runs_out_and_is_reported(hooks, monkeypatch, segments):
    import kla_b200

    if segments is not None:
        monkeypatch.setenv("KLA_B200_SEGMENTS", str(segments))
    ins = _inputs(False)
    with torch.no_grad():
        y0, yv0, st0 = kla_b200.kla_scan_b200(*ins)
    assert L.device_status() == 0
    assert hooks.kla_b200_test_hooks(3_000_000, 1) == 0  # 3 ms; tile 1 (steps 16..31) is never handed over
    with torch.no_grad():
        kla_b200.kla_scan_b200(*ins)
    torch.cuda.synchronize()  # the kernel returned
    with pytest.raises(RuntimeError, match="bounded wait"):
        L.check_status()
    assert hooks.kla_b200_test_hooks(3_000_000, 1) == 0
    with torch.no_grad():
        kla_b200.kla_scan_b200(*ins)
    st = L.device_status()
    # whoever waits for that tile first records it: the compute warps (site 1) or the storing warps (site 4)
    assert st & 0x100 and (st & 0xFF) in ((1, 4) if segments is None else (1, 4, 9)), hex(st)
    assert L.device_status() == 0, "reading the status clears it"
    assert hooks.kla_b200_test_hooks(0, -1) == 0
    with torch.no_grad():
        y1, yv1, st1 = kla_b200.kla_scan_b200(*ins)
    assert torch.equal(y1, y0) and torch.equal(yv1, yv0) and torch.equal(st1.lam, st0.lam)
    assert L.device_status() == 0


@pytest.mark.parametrize("segments", [None, 3])
def test_backward_wait_runs_out_and_is_reported(hooks, monkeypatch, segments):
    import kla_b200

    if segments is not None:
        monkeypatch.setenv("KLA_B200_SEGMENTS", str(segments))
    ins = _inputs(True)
    y, yv, _ = kla_b200.kla_scan_b200(*ins)
    good = torch.autograd.grad((y.square().sum() + yv.sum()), ins, retain_graph=True)
    assert L.device_status() == 0
    assert hooks.kla_b200_test_hooks(3_000_000, 2) == 0
    torch.autograd.grad((y.square().sum() + yv.sum()), ins, retain_graph=True)
    st = L.device_status()
    # whoever waits on that tile first: the replay warps on its inputs (site 11), the reverse warps on its
    # trajectory (17) or inputs (18), the summing warps on its partial sums (14)
    assert st & 0x100 and (st & 0xFF) in ((11, 14, 17, 18) if segments is None else (11, 14, 17, 18, 19)), hex(st)
    assert hooks.kla_b200_test_hooks(0, -1) == 0
    again = torch.autograd.grad((y.square().sum() + yv.sum()), ins)
    for g0, g1, n in zip(good, again, "v lambda_v k q a p".split()):
        # dk, dq, da, dp are sums by atomic adds, whose order may differ from launch to launch
        torch.testing.assert_close(g1, g0, rtol=1e-5, atol=1e-6, msg=lambda m: f"d{n}: {m}")
    assert L.device_status() == 0
