"""Host-side logic on the CPU: error behaviour of the backend callable, the
wrapper's plumbing with the kernel launches replaced by the oracle, plugging
into the reference package, and the batch x channel sharding under gloo."""

import importlib
import os
import sys

import numpy as np
import pytest
import torch

from conftest import load_golden, reference_src
from oracle import kla_oracle as O

import kla_b200

ops = importlib.import_module("kalman-linear-attention_b200.ops")
REF_SRC = reference_src()  # the directory holding the reference package `kla`, or "" when there is none here
INPUTS = ("v", "lambda_v", "k", "q", "a", "p")


def _t(g, names=INPUTS, dtype=torch.float32):
    return [torch.tensor(g[n], dtype=dtype) for n in names]


# ------------------------------------------------------------ error behaviour

def test_cpu_tensors_are_refused_not_served():
    ins = _t(load_golden("backends"))
    with pytest.raises(NotImplementedError, match="backend='torch'"):
        kla_b200.kla_scan_b200(*ins)
    with pytest.raises(NotImplementedError, match="CUDA"):
        kla_b200.kla_step_b200(ins[0][:, 0], ins[1][:, 0], ins[2][:, 0], ins[3][:, 0], ins[4], ins[5],
                               kla_b200.init_state(2, 16, 8))


# ----------------------------------- wrapper plumbing with oracle-backed launches

@pytest.fixture
def oracle_launches(monkeypatch):
    """Replace the two kernel launches by the CPU oracle and let CPU tensors
    through, so that everything above the C-ABI call runs here."""
    monkeypatch.setattr(ops, "_require_device", lambda t: None)

    def precision(x, sensors):  # the sensor prologue, src/kla/layers/kla_layer.py:224-231, and its slope
        sig = np.logaddexp(0.0, x) + sensors[0]
        free = np.ones_like(sig) if sensors[1] is None else (sig < sensors[1]).astype(np.float64)
        if sensors[1] is not None:
            sig = np.minimum(sig, sensors[1])
        return 1.0 / sig, -free / (sig * sig) / (1.0 + np.exp(-x))

    def fwd(v, lambda_v, k, q, a, p, lam0, eta0, prior, out_dtype, need_ckpt, sensors=None, epilogue=None, raw=None):
        n = lambda t: None if t is None else t.detach().double().numpy()
        lv = n(lambda_v) if sensors is None else precision(n(lambda_v), sensors)[0]
        f = O.scan_fwd(n(v), lv, n(k), n(q), n(a), n(p), n(lam0), n(eta0), prior=prior)
        return (torch.tensor(f.y, dtype=out_dtype), torch.tensor(f.y_var, dtype=out_dtype),
                torch.tensor(f.lam, dtype=torch.float32), torch.tensor(f.eta, dtype=torch.float32),
                torch.zeros(1, dtype=torch.uint8) if need_ckpt else None)

    def bwd(v, lambda_v, k, q, a, p, lam0, eta0, ckpt, dy, dy_var, dlam_fin, deta_fin, prior, out_dtype, sensors=None):
        n = lambda t: None if t is None else t.detach().double().numpy()
        lv, slope = (n(lambda_v), 1.0) if sensors is None else precision(n(lambda_v), sensors)
        g = O.scan_bwd(n(v), lv, n(k), n(q), n(a), n(p), n(dy), n(dy_var), n(lam0), n(eta0),
                       n(dlam_fin), n(deta_fin), prior=prior)
        f32 = lambda x, dt=torch.float32: torch.tensor(x, dtype=dt)
        return (f32(g.dv, v.dtype), f32(g.dlambda_v * slope, v.dtype), f32(g.dk), f32(g.dq), f32(g.da), f32(g.dp),
                f32(g.dlam0), f32(g.deta0))

    monkeypatch.setattr(ops, "_launch_fwd", fwd)
    monkeypatch.setattr(ops, "_launch_bwd", bwd)


def test_wrapper_contract(oracle_launches):
    g = load_golden("backends_state_prior")
    ins = [t.requires_grad_(True) for t in _t(g)]
    lam0 = torch.tensor(g["lam0"], dtype=torch.float32, requires_grad=True)
    eta0 = torch.tensor(g["eta0"], dtype=torch.float32, requires_grad=True)
    y, y_var, st = kla_b200.kla_scan_b200(*ins, initial_state=(lam0, eta0), decode_from_prior=True)
    assert y.dtype == torch.float32 and y.shape == ins[0].shape
    assert hasattr(st, "lam") and hasattr(st, "eta")
    loss = ((y * torch.tensor(g["dy"], dtype=torch.float32)).sum()
            + (y_var * torch.tensor(g["dyvar"], dtype=torch.float32)).sum()
            + (st.lam * torch.tensor(g["dlam_fin"], dtype=torch.float32)).sum()
            + (st.eta * torch.tensor(g["deta_fin"], dtype=torch.float32)).sum())
    grads = torch.autograd.grad(loss, ins + [lam0, eta0])
    for n, gr in zip(["dv", "dlambda_v", "dk", "dq", "da", "dp", "dlam0", "deta0"], grads):
        np.testing.assert_allclose(gr.numpy(), g[n], rtol=2e-4, atol=2e-5, err_msg=n)


def test_wrapper_passes_the_sensor_prologue_through(oracle_launches):
    """log_variance=(floor, ceiling): the second argument is the raw log-variance, and its gradient is with
    respect to that; both must equal the explicit torch prologue in front of the plain call."""
    g = load_golden("backends")
    ins = _t(g)
    x = torch.randn(ins[1].shape, generator=torch.Generator().manual_seed(5)).requires_grad_(True)
    for sensors in ((1e-4, None), (0.05, 1.2)):
        leaves = [t.clone().requires_grad_(True) for t in (ins[0], x, *ins[2:])]
        y, y_var, _ = kla_b200.kla_scan_b200(*leaves, log_variance=sensors)
        got = torch.autograd.grad((y.square().sum() + y_var.sum()), leaves)
        ref_leaves = [t.clone().requires_grad_(True) for t in (ins[0], x, *ins[2:])]
        sig = torch.nn.functional.softplus(ref_leaves[1]) + sensors[0]
        if sensors[1] is not None:
            sig = sig.clamp_max(sensors[1])
        y2, y_var2, _ = kla_b200.kla_scan_b200(ref_leaves[0], 1.0 / sig, *ref_leaves[2:])
        ref = torch.autograd.grad((y2.square().sum() + y_var2.sum()), ref_leaves)
        torch.testing.assert_close(y, y2, rtol=1e-5, atol=1e-6)
        for a_, b_ in zip(got, ref):
            torch.testing.assert_close(a_, b_, rtol=1e-4, atol=1e-5)
    with pytest.raises(ValueError, match="log_variance"):
        kla_b200.kla_scan_b200(*ins, log_variance=(-1.0, None))


def test_wrapper_widens_and_validates(oracle_launches):
    g = load_golden("backends")
    ins = _t(g)
    # half precision is widened to float32 like the reference (kla_ops.py:126-137)
    y, _, _ = kla_b200.kla_scan_b200(*[t.half() if i < 4 else t for i, t in enumerate(ins)])
    assert y.dtype == torch.float32
    # bfloat16 activations stay bfloat16 into the kernel; outputs are float32 unless asked
    y, _, _ = kla_b200.kla_scan_b200(*[t.bfloat16() if i < 4 else t for i, t in enumerate(ins)])
    assert y.dtype == torch.float32
    y, _, _ = kla_b200.kla_scan_b200(*[t.bfloat16() if i < 4 else t for i, t in enumerate(ins)],
                                      out_dtype=torch.bfloat16)
    assert y.dtype == torch.bfloat16
    with pytest.raises(NotImplementedError, match="float32 only"):
        kla_b200.kla_scan_b200(*[t.double() for t in ins])
    with pytest.raises(NotImplementedError, match=r"\[M, S\]"):
        kla_b200.kla_scan_b200(*ins[:4], ins[4][None], ins[5][None])
    with pytest.raises(NotImplementedError, match="d_state <= 128"):
        B, L = 1, 2
        kla_b200.kla_scan_b200(torch.zeros(B, L, 2), torch.ones(B, L, 2), torch.zeros(B, L, 129),
                               torch.zeros(B, L, 129), torch.ones(2, 129), torch.ones(2, 129))
    with pytest.raises(ValueError):
        kla_b200.kla_scan_b200(ins[0], ins[1][:, :-1], *ins[2:])
    # a non-unit last stride is copied, a row-strided view is passed through
    wide = torch.zeros(2, 64, 40)
    wide[..., 3:19] = ins[0]
    y2, _, _ = kla_b200.kla_scan_b200(wide[..., 3:19], *ins[1:])
    y1, _, _ = kla_b200.kla_scan_b200(*ins)
    torch.testing.assert_close(y1, y2)


# ------------------------------------------------ plugging into the reference

needs_ref = pytest.mark.skipif(not os.path.isdir(REF_SRC), reason="reference package not present")


@needs_ref
def test_register_into_reference_dispatch(oracle_launches):
    sys.path.insert(0, REF_SRC)
    try:
        import kla
        from kla.ops import kla_ops

        before_auto = kla_ops._resolve_auto(torch.zeros(1))
        kla_b200.register()
        try:
            assert "b200" in kla.ops.backend_names()
            assert kla_ops._resolve_auto(torch.zeros(1)) == before_auto  # "auto" untouched
            g = load_golden("backends")
            ins = _t(g)
            y, y_var, st = kla.ops.kla_scan(*ins, backend="b200")
            assert isinstance(st, kla_ops.KLAState)
            y_ref, _, _ = kla.ops.kla_scan_reference(*ins)
            torch.testing.assert_close(y, y_ref, atol=2e-4, rtol=1e-4)
            # through the layer: KLAConfig(backend="b200") reaches the callable
            torch.manual_seed(0)
            layer = kla.KLALayer(32, kla.KLAConfig(d_state=8, backend="b200"))
            ref = kla.KLALayer(32, kla.KLAConfig(d_state=8, backend="torch"))
            ref.load_state_dict(layer.state_dict())
            x = torch.randn(2, 24, 32)
            torch.testing.assert_close(layer(x), ref(x), atol=5e-4, rtol=5e-4)
            # the decode hook leaves CPU tensors to the original kla_step
            import kla.layers.kla_layer as kl

            assert kl.kla_step is not kla_ops.kla_step
            out = kl.kla_step(ins[0][:, 0], ins[1][:, 0], ins[2][:, 0], ins[3][:, 0], ins[4], ins[5],
                              kla_ops.init_state(2, 16, 8))
            ref_out = kla_ops.kla_step(ins[0][:, 0], ins[1][:, 0], ins[2][:, 0], ins[3][:, 0], ins[4], ins[5],
                                       kla_ops.init_state(2, 16, 8))
            torch.testing.assert_close(out[0], ref_out[0])
        finally:
            kla_b200.unregister()
        assert "b200" not in kla.ops.backend_names()
        with pytest.raises(ValueError):
            kla.ops.kla_scan(*_t(load_golden("backends")), backend="b200")
    finally:
        sys.path.remove(REF_SRC)


@needs_ref
def test_fused_layer_route_on_cpu(oracle_launches):
    """layer.fused_forward with oracle-backed launches: a layer without convolution, gate and skip path (the parts
    that need the GPU kernels) gives the reference layer's output and parameter gradients; and with the route
    enabled, CPU tensors still go to the reference method."""
    sys.path.insert(0, REF_SRC)
    try:
        import kla

        fused = importlib.import_module("kalman-linear-attention_b200.layer")
        cfg = dict(d_state=8, use_conv=False, use_gating=False, use_lambda_skip=False, obs_var_max=2.0)
        torch.manual_seed(0)
        ref = kla.KLALayer(32, kla.KLAConfig(backend="torch", **cfg))
        dut = kla.KLALayer(32, kla.KLAConfig(backend="b200", **cfg))
        dut.load_state_dict(ref.state_dict())
        x = torch.randn(2, 20, 32)
        y_ref = ref(x)
        y_ref.square().sum().backward()
        y, st = fused.fused_forward(dut, x, return_state=True)
        y.square().sum().backward()
        torch.testing.assert_close(y, y_ref, atol=5e-4, rtol=5e-4)
        assert st.conv is None and st.ssm.lam.shape == (2, 64, 8)
        grads = dict(dut.named_parameters())
        for n, p in ref.named_parameters():
            if p.grad is not None:
                torch.testing.assert_close(grads[n].grad, p.grad, atol=2e-3, rtol=2e-3, msg=lambda m, n=n: f"{n}: {m}")
        # enabled, but not applicable to CPU tensors: the reference method runs (and reaches the b200 callable)
        kla_b200.register(fuse_layer=True)
        try:
            assert not fused._fusable(dut, x, None)
            torch.testing.assert_close(dut(x), y.detach(), atol=1e-5, rtol=1e-5)
        finally:
            kla_b200.unregister()
        assert kla.KLALayer.forward is fused._ORIG_FORWARD or fused._ORIG_FORWARD is None
    finally:
        sys.path.remove(REF_SRC)


@needs_ref
def test_cli_rows_for_the_reference_command_line(capsys):
    """`python -m kla --check-backends` with the b200 row added: listed, described, and reported
    unusable on a machine without a CUDA device (src/kla/__main__.py:104-150, :290-300)."""
    pytest.importorskip("tyro")
    sys.path.insert(0, REF_SRC)
    try:
        import kla.__main__ as kla_main
        from importlib import import_module

        cli = import_module("kalman-linear-attention_b200.cli")
        try:
            assert cli.main(["--check-backends"]) == 0
            out = capsys.readouterr().out
            row = [ln for ln in out.splitlines() if " b200 " in ln]
            assert len(row) == 1 and "sm_100a" in row[0]
            if not torch.cuda.is_available():
                assert row[0].lstrip().startswith("[ ]") and "needs a CUDA device" in row[0]
                # the reference's own checks run the backend and report its refusal as a skip, not a crash
                assert cli.main(["--test-backends", "b200"]) == 1
                assert "skipped" in capsys.readouterr().out
            assert "b200" in kla_main._requirements() and kla_main._MODULES["b200"] == "kla_b200"
            cli.install_rows()  # idempotent
            assert getattr(kla_main._requirements, "_kla_b200", False)
        finally:
            kla_b200.unregister()
    finally:
        sys.path.remove(REF_SRC)


# ------------------------------------------------------------------- sharding

def test_blocks_tile_the_lane_grid():
    sh = kla_b200.shard
    for B, M, world in ((8, 1024, 1), (8, 1024, 2), (8, 1024, 8), (2, 4096, 8), (3, 100, 4), (16, 1536, 8)):
        seen = np.zeros((B, M), int)
        for r in range(world):
            blk = sh.block_of(B, M, world, r)
            seen[blk.b0:blk.b1, blk.m0:blk.m1] += 1
            assert blk.batch_parts * blk.channel_parts == world
        assert (seen == 1).all(), (B, M, world)
    assert sh.grid_for(8, 1024, 8) == (8, 1)   # batch first
    assert sh.grid_for(2, 4096, 8) == (2, 4)   # then channels
    blk = sh.block_of(2, 4096, 8, 5)
    assert (blk.m1 - blk.m0) % 32 == 0


def _worker(rank, world, port, case, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        opsm = importlib.import_module("kalman-linear-attention_b200.ops")
        sh = kla_b200.shard

        class CpuScan(torch.autograd.Function):  # oracle-backed stand-in for the kernels
            @staticmethod
            def forward(ctx, v, lv, k, qq, a, p):
                n = lambda t: t.detach().double().numpy()
                f = O.scan_fwd(n(v), n(lv), n(k), n(qq), n(a), n(p))
                ctx.save_for_backward(v, lv, k, qq, a, p)
                return torch.tensor(f.y), torch.tensor(f.y_var)

            @staticmethod
            def backward(ctx, dy, dyv):
                n = lambda t: t.detach().double().numpy()
                g = O.scan_bwd(*[n(t) for t in ctx.saved_tensors], n(dy), n(dyv))
                return tuple(torch.tensor(x) for x in (g.dv, g.dlambda_v, g.dk, g.dq, g.da, g.dp))

        def scan_fn(v, lv, k, qq, a, p, initial_state=None, decode_from_prior=False):
            y, yv = CpuScan.apply(v, lv, k, qq, a, p)
            return y, yv, None

        g = load_golden("cfg2small")
        full = [torch.tensor(g[n]).requires_grad_(True) for n in INPUTS]
        B, M = (2, 24) if case == "batch" else (1, 24)
        if case == "channel":
            full = [t[:1].detach().requires_grad_(True) if t.dim() == 3 else t for t in full]
        blk = sh.block_of(B, M, world, rank, align=4)
        groups = sh.make_groups(world, blk.batch_parts, blk.channel_parts)
        v, lv, k, qq, a, p, _ = sh.take_block(blk, *full)
        y, yv, _ = sh.scan_block(scan_fn, groups, v, lv, k, qq, a, p)
        dy = torch.tensor(g["dy"])[blk.b0:blk.b1, :, blk.m0:blk.m1]
        dyv = torch.tensor(g["dyvar"])[blk.b0:blk.b1, :, blk.m0:blk.m1]
        grads = torch.autograd.grad((y * dy).sum() + (yv * dyv).sum(), full)
        q.put((rank, tuple(blk), y.detach().numpy(), [t.numpy() for t in grads]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("case", ["batch", "channel"])
def test_sharded_scan_matches_full_under_gloo(case):
    """world_size 2 on CPU: the blocks' outputs tile the full output, and after
    the backward's all-reduces every rank holds the full-problem da, dp (batch
    split) or dk, dq (channel split)."""
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000) + (0 if case == "batch" else 1)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, case, q)) for r in range(2)]
    [p.start() for p in procs]
    res = sorted([q.get(timeout=120) for _ in procs], key=lambda t: t[0])
    [p.join(timeout=60) for p in procs]
    assert all(p.exitcode == 0 for p in procs)

    g = load_golden("cfg2small")
    ins = [g[n] for n in INPUTS]
    dy, dyv = g["dy"], g["dyvar"]
    if case == "channel":
        ins = [x[:1] if x.ndim == 3 else x for x in ins]
        dy, dyv = dy[:1], dyv[:1]
    f = O.scan_fwd(*ins)
    b = O.scan_bwd(*ins, dy, dyv)
    for rank, blk, y, grads in res:
        b0, b1, m0, m1 = blk[:4]
        np.testing.assert_allclose(y, f.y[b0:b1, :, m0:m1], rtol=1e-10, atol=1e-12)
        dv, dlv, dk, dq, da, dp = grads
        # autograd wrote each rank's slice of the full-shaped gradient
        np.testing.assert_allclose(dv[b0:b1, :, m0:m1], b.dv[b0:b1, :, m0:m1], rtol=1e-9, atol=1e-12)
        np.testing.assert_allclose(dk[b0:b1], b.dk[b0:b1], rtol=1e-9, atol=1e-11)   # summed over channels
        np.testing.assert_allclose(da[m0:m1], b.da[m0:m1], rtol=1e-9, atol=1e-11)   # summed over batch
        np.testing.assert_allclose(dp[m0:m1], b.dp[m0:m1], rtol=1e-9, atol=1e-11)


# --------------------------------------------------------- sequence sharding

def test_slab_folds_reproduce_the_scan_on_cpu():
    """The fold algebra alone, in numpy: slab aggregates folded onto the initial
    state give the state the oracle reaches; adjoint aggregates folded onto the
    final-state gradient give the carry the oracle's backward hands on."""
    import slab_math

    ss = kla_b200.seqshard
    g = load_golden("cfg2small")
    ins = [g[n] for n in INPUTS]
    v, lv, k, q, a, p = ins
    cuts = (0, 50, 111, 160)
    slabs = [slice(cuts[i], cuts[i + 1]) for i in range(3)]
    aggs = [torch.tensor(slab_math.forward_aggregate(v[:, s], lv[:, s], k[:, s], a, p)) for s in slabs]
    lam0, eta0 = torch.tensor(g["lam0"]), torch.tensor(g["eta0"])
    for r in range(1, 4):
        lam, eta = ss.prefix_state(aggs[:r], lam0, eta0, lam0.shape, "cpu")
        t1 = cuts[r]
        f = O.scan_fwd(v[:, :t1], lv[:, :t1], k[:, :t1], q[:, :t1], a, p, g["lam0"], g["eta0"])
        np.testing.assert_allclose(lam.numpy(), f.lam, rtol=2e-6)
        np.testing.assert_allclose(eta.numpy(), f.eta, rtol=2e-5, atol=1e-6)
    # carry handed from slab 1 to slab 0 == gradient of slab 1's initial state in the oracle
    f0 = O.scan_fwd(v[:, slabs[0]], lv[:, slabs[0]], k[:, slabs[0]], q[:, slabs[0]], a, p, g["lam0"], g["eta0"])
    tail = slice(cuts[1], cuts[3])
    b_tail = O.scan_bwd(v[:, tail], lv[:, tail], k[:, tail], q[:, tail], a, p, g["dy"][:, tail], g["dyvar"][:, tail],
                        f0.lam, f0.eta, g["dlam_fin"], g["deta_fin"])
    states = [(f0.lam, f0.eta)]
    f1 = O.scan_fwd(v[:, slabs[1]], lv[:, slabs[1]], k[:, slabs[1]], q[:, slabs[1]], a, p, f0.lam, f0.eta)
    states.append((f1.lam, f1.eta))
    f2 = O.scan_fwd(v[:, slabs[2]], lv[:, slabs[2]], k[:, slabs[2]], q[:, slabs[2]], a, p, f1.lam, f1.eta)
    adjs = [torch.tensor(slab_math.adjoint_aggregate(v[:, s], lv[:, s], k[:, s], q[:, s], a, p, g["dy"][:, s],
                                                     g["dyvar"][:, s], *st))
            for s, st in zip(slabs[1:], states)]
    P_end = torch.tensor(1.0 / f2.lam)
    cP, cm = ss.carry_from_state_grad(torch.tensor(g["dlam_fin"]), torch.tensor(g["deta_fin"]), P_end,
                                      torch.tensor(f2.eta) * P_end)
    cP, cm = ss.suffix_carry(adjs, cP, cm)
    # express the carry as a gradient of (lam, eta) at the end of slab 0 and compare
    P0 = torch.tensor(1.0 / f0.lam)
    dlam, deta = ss.state_grad_from_carry(cP, cm, P0, torch.tensor(f0.eta) * P0)
    np.testing.assert_allclose(dlam.numpy(), b_tail.dlam0, rtol=1e-7, atol=1e-9)
    np.testing.assert_allclose(deta.numpy(), b_tail.deta0, rtol=1e-7, atol=1e-9)


def _seq_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist

    import slab_math

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        opsm = importlib.import_module("kalman-linear-attention_b200.ops")
        ss = kla_b200.seqshard
        n = lambda t: None if t is None else t.detach().double().numpy()

        def fwd(v, lv, k, qq, a, p, lam0, eta0, prior, out_dtype, need_ckpt):
            f = O.scan_fwd(n(v), n(lv), n(k), n(qq), n(a), n(p), n(lam0), n(eta0), prior=prior)
            return (torch.tensor(f.y), torch.tensor(f.y_var), torch.tensor(f.lam), torch.tensor(f.eta), None)

        def bwd(v, lv, k, qq, a, p, lam0, eta0, ckpt, dy, dyv, dl, de, prior, out_dtype):
            b = O.scan_bwd(n(v), n(lv), n(k), n(qq), n(a), n(p), n(dy), n(dyv), n(lam0), n(eta0), n(dl), n(de),
                           prior=prior)
            return tuple(torch.tensor(x) for x in b)

        def agg(v, lv, k, a, p, *, q=None, dy=None, dy_var=None, lam0=None, eta0=None, prior=False):
            if dy is None:
                return torch.tensor(slab_math.forward_aggregate(n(v), n(lv), n(k), n(a), n(p)))
            return torch.tensor(slab_math.adjoint_aggregate(n(v), n(lv), n(k), n(q), n(a), n(p), n(dy), n(dy_var),
                                                            n(lam0), n(eta0), prior))

        opsm._launch_fwd, opsm._launch_bwd, ss.slab_aggregate = fwd, bwd, agg
        opsm._require_device = lambda t: None
        g = load_golden("cfg2small")
        cuts = (0, 70, 160)
        sl = slice(cuts[rank], cuts[rank + 1])
        full = [torch.tensor(g[k_]).requires_grad_(True) for k_ in INPUTS]
        lam0 = torch.tensor(g["lam0"]).requires_grad_(True)
        eta0 = torch.tensor(g["eta0"]).requires_grad_(True)
        v, lv, k, qq, a, p = full
        ins = (v[:, sl], lv[:, sl], k[:, sl], qq[:, sl], a, p)
        y, yv, lam, eta = ss._SeqShardedScan.apply(*ins, lam0, eta0, False, torch.float64, None)
        loss = (y * torch.tensor(g["dy"])[:, sl]).sum() + (yv * torch.tensor(g["dyvar"])[:, sl]).sum()
        if rank == world - 1:  # the state's gradient enters on one rank only
            loss = loss + (lam * torch.tensor(g["dlam_fin"])).sum() + (eta * torch.tensor(g["deta_fin"])).sum()
        grads = torch.autograd.grad(loss, full + [lam0, eta0])
        q.put((rank, (sl.start, sl.stop), y.detach().numpy(), lam.detach().numpy(), [t.numpy() for t in grads]))
    finally:
        dist.destroy_process_group()


def test_sequence_sharded_scan_under_gloo():
    """world_size 2 on CPU with the kernels replaced by the oracle and the numpy
    aggregates: checks the collectives and folds of the autograd function."""
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_seq_worker, args=(r, 2, port, q)) for r in range(2)]
    [p.start() for p in procs]
    res = sorted([q.get(timeout=180) for _ in procs], key=lambda t: t[0])
    [p.join(timeout=60) for p in procs]
    assert all(p.exitcode == 0 for p in procs)
    g = load_golden("cfg2small")
    ins = [g[n] for n in INPUTS]
    f = O.scan_fwd(*ins, g["lam0"], g["eta0"])
    b = O.scan_bwd(*ins, g["dy"], g["dyvar"], g["lam0"], g["eta0"], g["dlam_fin"], g["deta_fin"])
    for rank, (t0, t1), y, lam, grads in res:
        # the folded state crosses the slab boundary in float32, as on the GPU
        np.testing.assert_allclose(y, f.y[:, t0:t1], rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(lam, f.lam, rtol=1e-5)  # every rank returns the last slab's posterior
        dv, dlv, dk, dq, da, dp, dlam0, deta0 = grads
        tol = dict(rtol=2e-4, atol=2e-5)
        np.testing.assert_allclose(dv[:, t0:t1], b.dv[:, t0:t1], **tol)
        np.testing.assert_allclose(dk[:, t0:t1], b.dk[:, t0:t1], **tol)
        np.testing.assert_allclose(da, b.da, **tol)       # all-reduced over the slabs
        np.testing.assert_allclose(dp, b.dp, **tol)
        np.testing.assert_allclose(dlam0, b.dlam0, **tol)  # broadcast from the first slab
        np.testing.assert_allclose(deta0, b.deta0, **tol)


# ------------------------------------------------------------ time-parallel form: the choice of the chunk count

def test_chunk_count_follows_the_shape():
    pick = ops.pick_time_chunks
    assert pick(8, 4096, 1024, 16) == 1          # the grid already fills the GPU
    assert pick(1, 4096, 1024, 16) == 16         # 32 CTAs: cut the sequence
    assert pick(1, 4096, 1024, 16, 1) == 1       # switched off
    assert pick(1, 100, 64, 16, 8) == 1          # chunks keep at least 64 steps
    assert pick(1, 1100, 64, 16, 8) == 5         # C divides L
    assert 4096 % pick(2, 4096, 512, 16) == 0
    v = torch.zeros(2, 8, 4)
    assert ops._chunkable(v, 2, 8) and not ops._chunkable(torch.zeros(2, 12, 4)[:, :8], 2, 8)
    c = ops._as_chunks(torch.arange(2 * 8 * 3.0).view(2, 8, 3), 4)
    assert c.shape == (8, 2, 3) and torch.equal(c[5], torch.arange(2 * 8 * 3.0).view(2, 8, 3)[1, 2:4])
