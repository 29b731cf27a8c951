"""Everything above the op boundary, on the GPU, with the reference's own code on top of the B200 kernels.

The reference package is read from ``baseline/_ref`` (put there, unmodified, by
``baseline/install_reference.py``); every test here skips when it is absent.

* the reference's parity matrix (its ``tests/test_backends.py``) run against a
  ``b200`` profile: its test functions are called as they are, with the profile
  and the device table extended at run time -- no reference file is edited;
* the reference's command line: ``--test-backends b200``;
* ``KLALayer(512, KLAConfig(d_state=16))`` forward + backward on the GPU with
  ``backend="b200"`` against the same layer with ``backend="torch"`` on the CPU,
  also under ``checkpoint_ssm`` (src/kla/layers/kla_layer.py:260-272);
* prefill then single-token decode with bf16 I/O against a one-shot scan;
* a ``SequenceModel`` training step with ``backend="b200"`` against ``backend="torch"``.
"""

import importlib
import importlib.util
import inspect
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, ROOT)
REF = os.path.join(ROOT, "baseline", "_ref")
HAVE_REF = os.path.isfile(os.path.join(REF, "kla", "__init__.py"))

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not HAVE_REF, reason="reference not installed under baseline/_ref")]


@pytest.fixture(scope="module")
def kla():
    if REF not in sys.path:
        sys.path.insert(0, REF)
    import kla as kla_pkg

    import kla_b200

    kla_b200.register()
    yield kla_pkg
    kla_b200.unregister()


# ------------------------------------------------------------ the reference's own parity matrix

def _load_matrix():
    """The reference's tests/test_backends.py as a module, with a b200 profile added to its tables."""
    if REF not in sys.path:
        sys.path.insert(0, REF)
    spec = importlib.util.spec_from_file_location("kla_ref_test_backends", os.path.join(REF, "tests", "test_backends.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    # exact gradients on all six inputs, state in and out: the accuracy contract of the reference's own
    # lane-form backends (src tests/test_backends.py:78-130), with the forward budget of its CUDA kernels
    mod.PROFILES["b200"] = mod.Profile("b200", 1e-4, 1e-4, exact_grads=mod.INPUT_NAMES, returns_state=True,
                                       supports_initial_state=True, scan_form=mod._LANE_FORM)
    mod._DEVICE["b200"] = "cuda"
    # the lane-form tests are written for the Metal device; the same tests apply to any lane-form backend
    make_inputs = mod.make_inputs
    mod.make_inputs = lambda device, *a, **kw: make_inputs("cuda" if device == "mps" else device, *a, **kw)
    return mod


_MATRIX_ALL = [  # every test the reference parametrises over ALL_BACKENDS (tests/test_backends.py:220-497)
    ("test_forward_matches_reference", {}),
    ("test_final_state_matches_reference", {}),
    ("test_chunked_state_carry", {}),
    ("test_backward_matches_reference", {}),
    ("test_gradient_descent_reduces_loss", {}),
    ("test_non_positive_process_noise_stays_finite", {"bad_p": 0.0}),
    ("test_non_positive_process_noise_stays_finite", {"bad_p": -0.05}),
    ("test_near_zero_decay_stays_finite", {}),
    ("test_high_information_tokens_are_not_clipped", {}),
]
_MATRIX_LANE = (  # the tests it keeps for its lane-form (Metal) backends (:697-964): tile boundaries, padding lanes, ...
    [("test_mps_chunk_boundaries", {"L": L}) for L in (1, 15, 16, 17, 32, 100)]
    + [("test_mps_threadgroup_geometry", {"S": S, "M": M}) for S in (1, 3, 16, 32, 33, 64) for M in (1, 33)]
    + [("test_mps_state_gradient_flows", {}), ("test_mps_decode_from_prior", {})]
    + [("test_mps_widens_low_precision_inputs", {"dtype": d}) for d in (torch.bfloat16, torch.float16)]
)


@pytest.mark.parametrize("name,kwargs", _MATRIX_ALL + _MATRIX_LANE,
                         ids=lambda x: x if isinstance(x, str) else "-".join(f"{k}={v}" for k, v in x.items()) or "-")
def test_reference_parity_matrix(kla, name, kwargs, capsys):
    mod = _load_matrix()
    fn = getattr(mod, name)
    fn = inspect.unwrap(fn)
    torch.manual_seed(0)  # the reference's autouse fixture, tests/conftest.py
    fn(backend="b200", **kwargs)
    out = capsys.readouterr().out
    if out.strip():
        with capsys.disabled():
            print(out)


def test_reference_coverage_guard_accepts_b200(kla):
    """tests/test_backends.py:986-998 fails for a dispatcher entry without a profile; with the profile it passes."""
    mod = _load_matrix()
    assert "b200" in kla.backend_names()
    mod.test_every_backend_is_covered()


def test_reference_cli_tests_b200():
    """``python -m kla --test-backends b200`` through the overlay (src/kla/__main__.py:158-263): exit 0, both rows ok."""
    env = dict(os.environ, PYTHONPATH=REF + os.pathsep + os.environ.get("PYTHONPATH", ""))
    res = subprocess.run([sys.executable, os.path.join(ROOT, "kla_b200.py"), "--test-backends", "b200"],
                         capture_output=True, text=True, env=env, timeout=600)
    print(res.stdout, res.stderr[-2000:])
    assert res.returncode == 0, res.stdout + res.stderr[-2000:]
    assert "forward    ok" in res.stdout and "gradients  ok" in res.stdout
    res = subprocess.run([sys.executable, os.path.join(ROOT, "kla_b200.py"), "--check-backends"],
                         capture_output=True, text=True, env=env, timeout=600)
    assert res.returncode == 0 and "[x] b200" in res.stdout.lower(), res.stdout + res.stderr[-2000:]


# ------------------------------------------------------------ KLALayer(512, d_state=16), x (2, 1024, 512)

def _rel(got, ref):
    return ((got - ref).abs().max() / (ref.abs().max() + 1.0)).item()


def _layer_pair(kla, d_model, seed=0, **cfg):
    from kla import KLAConfig, KLALayer

    torch.manual_seed(seed)
    ref = KLALayer(d_model, KLAConfig(d_state=16, backend="torch", **cfg))
    dut = KLALayer(d_model, KLAConfig(d_state=16, backend="b200", **cfg))
    dut.load_state_dict(ref.state_dict())
    return ref, dut.cuda()


@pytest.mark.parametrize("checkpoint_ssm", [False, True])
def test_layer_forward_backward_matches_cpu_torch_backend(kla, checkpoint_ssm):
    ref, dut = _layer_pair(kla, 512, checkpoint_ssm=checkpoint_ssm)
    names = [n for n, _ in ref.named_parameters()]
    assert len(names) == 9 and sum(p.numel() for p in ref.parameters()) == 3_757_057
    torch.manual_seed(0)
    x = torch.randn(2, 1024, 512)
    ref.train(); dut.train()
    y_ref = ref(x)
    y_ref.square().sum().backward()
    launches0 = importlib.import_module("kalman-linear-attention_b200._lib").load().kla_b200_launch_count()
    y = dut(x.cuda())
    y.square().sum().backward()
    torch.cuda.synchronize()
    launches = importlib.import_module("kalman-linear-attention_b200._lib").load().kla_b200_launch_count() - launches0
    # forward + backward, and the forward once more when the scan is recomputed under checkpointing; at this shape
    # (2 x 1024 channels) the scan runs time-parallel: aggregate, fold and scan kernel in each direction
    ops = importlib.import_module("kalman-linear-attention_b200.ops")
    per = 3 if ops.pick_time_chunks(2, 1024, 1024, 16) > 1 else 1
    assert launches == per * (3 if checkpoint_ssm else 2), launches
    rows = [("y", _rel(y.cpu(), y_ref))]
    torch.testing.assert_close(y.cpu(), y_ref, rtol=1e-4, atol=1e-5)
    gp = dict(dut.named_parameters())
    for n, p in ref.named_parameters():
        assert gp[n].grad is not None, n
        rows.append((n, _rel(gp[n].grad.cpu(), p.grad)))
    print("\n  KLALayer(512, d_state=16) b200 on GPU vs torch backend on CPU, checkpoint_ssm =", checkpoint_ssm)
    for n, e in rows:
        print(f"    {n:<22} {e:.2e}")
    bad = [(n, e) for n, e in rows if not e < 2e-3]  # the reference's gradient contract, tests/test_backends.py:54
    assert not bad, bad


@pytest.fixture()
def fused_layers(kla):
    """KLALayer.forward routed through the fused path for the duration of a test."""
    layer = importlib.import_module("kalman-linear-attention_b200.layer")
    layer.enable()
    yield layer
    layer.disable()


_FUSED_CONFIGS = {
    "default": {},
    "checkpointed": dict(checkpoint_ssm=True),
    "value_from_conv": dict(value_rank="conv"),
    "low_rank_sensors": dict(value_rank=24, var_rank="dt"),
    "vector_skip_gelu_gate": dict(lambda_skip_mode="vector", gating_activation="gelu"),
    "bare": dict(use_gating=False, use_lambda_skip=False, use_conv=False, qk_norm=False),
    "variance_out_prior_readout": dict(return_variance=True, decode_from_prior=True),
}


@pytest.mark.parametrize("name", list(_FUSED_CONFIGS))
def test_fused_layer_forward_backward_matches_cpu_torch_backend(kla, fused_layers, name):
    """layer.fused_forward (sensor prologue and skip/gate epilogue inside the scan kernels) against the reference
    layer on its torch backend on the CPU: output(s) and every parameter gradient, float32."""
    cfg = _FUSED_CONFIGS[name]
    ref, dut = _layer_pair(kla, 256, **cfg)
    torch.manual_seed(0)
    x = torch.randn(2, 200, 256)
    ref.train(); dut.train()

    def loss(out):
        return sum(o.square().sum() for o in out) if isinstance(out, tuple) else out.square().sum()

    out_ref = ref(x)
    loss(out_ref).backward()
    lib = importlib.import_module("kalman-linear-attention_b200._lib").load()
    n0 = lib.kla_b200_launch_count()
    xg = x.cuda().requires_grad_(True)
    out = dut(xg)
    loss(out).backward()
    torch.cuda.synchronize()
    assert lib.kla_b200_launch_count() > n0
    pairs = list(zip(out, out_ref)) if isinstance(out, tuple) else [(out, out_ref)]
    for got, want in pairs:
        torch.testing.assert_close(got.detach().cpu(), want.detach(), rtol=1e-4, atol=1e-5)
    gp = dict(dut.named_parameters())
    bad = []
    for n, p in ref.named_parameters():
        if p.grad is None:
            assert gp[n].grad is None, n
            continue
        assert gp[n].grad is not None, n
        e = _rel(gp[n].grad.cpu(), p.grad)
        if not e < 2e-3:
            bad.append((n, e))
    assert not bad, bad


def test_fused_layer_is_the_route_taken_and_saves_elementwise_kernels(kla, fused_layers):
    """With the route enabled a b200 layer launches fewer kernels than the same layer on the reference's forward,
    returns the same state, and leaves layers of other backends and the single-token route alone."""
    from torch.profiler import ProfilerActivity, profile

    ref, dut = _layer_pair(kla, 128)
    dut.eval()
    x = torch.randn(2, 64, 128).cuda()

    def kernels(fn):
        fn(); torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            fn(); torch.cuda.synchronize()
        return sum(e.count for e in prof.key_averages() if e.device_time_total > 0)

    with torch.no_grad():
        n_fused = kernels(lambda: dut(x))
        (out, st) = dut(x, return_state=True)
        fused_layers.disable()
        n_plain = kernels(lambda: dut(x))
        (out0, st0) = dut(x, return_state=True)
        fused_layers.enable()
        o1, st1 = dut(x[:, :1], state=st)          # decode by one token: the reference method with the step kernel
        fused_layers.disable()
        o2, st2 = dut(x[:, :1], state=st0)
        fused_layers.enable()
    assert n_fused < n_plain, (n_fused, n_plain)
    torch.testing.assert_close(out, out0, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(st.ssm.lam, st0.ssm.lam, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(st.ssm.eta, st0.ssm.eta, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(st.conv, st0.conv)
    torch.testing.assert_close(o1, o2, rtol=1e-5, atol=1e-6)


def test_fused_layer_under_bf16_autocast_tracks_the_unfused_route(kla, fused_layers):
    """Under bf16 autocast the fused route reads the projections' bf16 slices directly and writes bf16; against the
    reference forward with the same backend (which widens to float32 around the scan) outputs and gradients agree
    to bf16 rounding."""
    ref, dut = _layer_pair(kla, 256)
    dut.train()
    torch.manual_seed(1)
    x = torch.randn(2, 256, 256).cuda()

    def run():
        dut.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y = dut(x)
        y.float().square().sum().backward()
        return y.detach().float(), {n: p.grad.detach().float().clone() for n, p in dut.named_parameters()}

    y_f, g_f = run()
    fused_layers.disable()
    y_u, g_u = run()
    fused_layers.enable()
    assert _rel(y_f, y_u) < 2e-2, _rel(y_f, y_u)
    bad = [(n, _rel(g_f[n], g_u[n])) for n in g_u if not _rel(g_f[n], g_u[n]) < 5e-2]
    assert not bad, bad


def test_fused_layer_in_a_bfloat16_model(kla, fused_layers):
    """Every parameter in bfloat16 (no autocast): gradients come back in the parameters' dtype and track the
    unfused route to bf16 rounding."""
    ref, dut = _layer_pair(kla, 256, lambda_skip_mode="vector")
    dut = dut.to(torch.bfloat16).train()
    torch.manual_seed(2)
    x = torch.randn(2, 128, 256, device="cuda", dtype=torch.bfloat16)

    def run():
        dut.zero_grad(set_to_none=True)
        y = dut(x)
        y.float().square().sum().backward()
        for n, p in dut.named_parameters():
            assert p.grad is not None and p.grad.dtype == p.dtype, n
        return y.detach().float(), {n: p.grad.detach().float().clone() for n, p in dut.named_parameters()}

    y_f, g_f = run()
    fused_layers.disable()
    y_u, g_u = run()
    fused_layers.enable()
    assert y_f.dtype == y_u.dtype and _rel(y_f, y_u) < 3e-2, _rel(y_f, y_u)
    bad = [(n, _rel(g_f[n], g_u[n])) for n in g_u if not _rel(g_f[n], g_u[n]) < 8e-2]
    assert not bad, bad


def test_layer_runs_under_autocast_and_no_grad(kla):
    """The layer switches autocast off around the scan (kla_layer.py:261) and hands it float32; bf16 autocast
    outside must therefore change nothing for the backend, and no_grad must not ask for checkpoints."""
    ref, dut = _layer_pair(kla, 128)
    x = torch.randn(2, 96, 128)
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        y = dut(x.cuda())
    with torch.no_grad(), torch.autocast("cpu", dtype=torch.bfloat16):
        y_ref = ref(x)
    assert y.dtype == y_ref.dtype
    torch.testing.assert_close(y.float().cpu(), y_ref.float(), rtol=5e-2, atol=5e-2)


def test_layer_decode_route_uses_the_step_kernel(kla):
    """With a state and L == 1 the layer calls the name kla_step it imported (kla_layer.py:277-293, 324-325);
    register() rebinds it. Prefill + 8 decoded tokens must equal the full-sequence forward."""
    ref, dut = _layer_pair(kla, 128)
    dut.eval()
    x = torch.randn(2, 40, 128).cuda()
    lib = importlib.import_module("kalman-linear-attention_b200._lib").load()
    with torch.no_grad():
        full = dut(x)
        out, st = dut(x[:, :32], state=dut.init_state(2, device="cuda"))
        outs = [out]
        n0 = lib.kla_b200_launch_count()
        for t in range(32, 40):
            o, st = dut(x[:, t:t + 1], state=st)
            outs.append(o)
        assert lib.kla_b200_launch_count() - n0 == 8  # one step kernel per token
    torch.testing.assert_close(torch.cat(outs, 1), full, rtol=1e-4, atol=1e-5)


# ------------------------------------------------------------ prefill + decode, bf16 I/O, against a one-shot scan

def test_prefill_then_decode_bf16_equals_one_shot_scan(kla):
    """B x (8192 + 256) tokens at M = 2048, S = 16, bf16 activations, float32 state: a prefill scan followed by 256
    single-token steps must leave the state a one-shot scan over all 8448 tokens leaves. The step kernel floors phi
    at 1e-12 like kla_step (kla_ops.py:310-312) and the scan does not (kla_ops.py:238), hence not bit-equality."""
    import kla_b200

    B, T, D, M, S = 3, 8192, 256, 2048, 16
    g = torch.Generator().manual_seed(0)
    bf = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).cuda()
    v = bf(B, T + D, M)
    lam_v = (1.0 / torch.nn.functional.softplus(torch.randn(B, T + D, M, generator=g))).to(torch.bfloat16).cuda()
    k = torch.nn.functional.normalize(torch.randn(B, T + D, S, generator=g), dim=-1).to(torch.bfloat16).cuda()
    q = torch.nn.functional.normalize(torch.randn(B, T + D, S, generator=g), dim=-1).to(torch.bfloat16).cuda()
    a = torch.sigmoid(torch.randn(M, S, generator=g)).cuda()
    p = torch.nn.functional.softplus(torch.randn(M, S, generator=g)).cuda()
    with torch.no_grad():
        y_all, yv_all, st_all = kla_b200.kla_scan_b200(v, lam_v, k, q, a, p, out_dtype=torch.bfloat16)
        y_pre, _, st = kla_b200.kla_scan_b200(v[:, :T], lam_v[:, :T], k[:, :T], q[:, :T], a, p, out_dtype=torch.bfloat16)
        ys = []
        for t in range(T, T + D):
            y_t, _, st = kla_b200.kla_step_b200(v[:, t], lam_v[:, t], k[:, t], q[:, t], a, p, st)
            ys.append(y_t)
    torch.testing.assert_close(st.lam, st_all.lam, rtol=2e-5, atol=1e-6)
    torch.testing.assert_close(st.eta, st_all.eta, rtol=2e-5, atol=2e-5)
    assert torch.equal(y_pre, y_all[:, :T])
    torch.testing.assert_close(torch.stack(ys, 1), y_all[:, T:].float(), rtol=2e-2, atol=2e-2)
    # and against the reference's own kla_step driven from the same prefill state, on a slice of channels
    sl = slice(0, 64)
    _, _, st0 = kla_b200.kla_scan_b200(v[:, :T, sl], lam_v[:, :T, sl], k[:, :T], q[:, :T], a[sl], p[sl])
    ref_state = kla.ops.KLAState(lam=st0.lam.cpu(), eta=st0.eta.cpu())
    from kla.ops.kla_ops import kla_step as ref_step  # the module attribute stays the reference's own

    for t in range(T, T + D):
        _, _, ref_state = ref_step(v[:, t, sl].float().cpu(), lam_v[:, t, sl].float().cpu(), k[:, t].float().cpu(),
                                   q[:, t].float().cpu(), a[sl].cpu(), p[sl].cpu(), ref_state)
    torch.testing.assert_close(st.lam[:, sl].cpu(), ref_state.lam, rtol=2e-5, atol=1e-6)
    torch.testing.assert_close(st.eta[:, sl].cpu(), ref_state.eta, rtol=2e-5, atol=2e-5)


# ------------------------------------------------------------ SequenceModel training step

@pytest.mark.parametrize("fused", [False, True])
def test_sequence_model_training_step_matches_torch_backend(kla, fused):
    """SequenceModel(ModelConfig(vocab 50304, d_model 768, 12 layers), KLAConfig(d_state=16)) on a short batch:
    loss and every parameter gradient with backend='b200' against backend='torch' (both on the GPU, float32);
    once with the reference's own layer forward, once with the layers routed through layer.fused_forward."""
    from kla import KLAConfig, ModelConfig, SequenceModel

    layer = importlib.import_module("kalman-linear-attention_b200.layer")
    if fused:
        layer.enable()
    try:
        _model_step_parity(KLAConfig, ModelConfig, SequenceModel)
    finally:
        layer.disable()


def _model_step_parity(KLAConfig, ModelConfig, SequenceModel):
    torch.manual_seed(0)
    mc = ModelConfig(vocab_size=50304, d_model=768, n_layers=12)
    ref = SequenceModel(mc, KLAConfig(d_state=16, backend="torch")).cuda()
    dut = SequenceModel(mc, KLAConfig(d_state=16, backend="b200")).cuda()
    dut.load_state_dict(ref.state_dict())
    ids = torch.randint(0, 50304, (2, 129), generator=torch.Generator().manual_seed(1)).cuda()

    def step(model):
        logits = model(ids[:, :-1])
        loss = torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), ids[:, 1:].reshape(-1))
        loss.backward()
        return loss

    l_ref, l_dut = step(ref), step(dut)
    torch.testing.assert_close(l_dut, l_ref, rtol=1e-5, atol=1e-5)
    gp = dict(dut.named_parameters())
    worst = ("", 0.0)
    for n, p in ref.named_parameters():
        e = _rel(gp[n].grad, p.grad)
        if e > worst[1]:
            worst = (n, e)
    print(f"\n  SequenceModel step: loss {l_dut.item():.6f} vs {l_ref.item():.6f}; worst gradient {worst[0]} {worst[1]:.2e}")
    assert worst[1] < 2e-3, worst


# ------------------------------------------------------------ multi-layer prefill + decode loop

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_model_decoder_generates_what_the_reference_generates(dtype):
    """``ModelDecoder`` (all layers on the fused decode kernels, the token loop as one CUDA graph) against the
    reference's own ``SequenceModel.generate`` on its torch backend (sequence_model.py:200-220): the prompt's logits,
    the per-token logits and, greedily, the generated tokens."""
    if REF not in sys.path:
        sys.path.insert(0, REF)
    import kla_b200
    from kla import KLAConfig, ModelConfig, SequenceModel

    torch.manual_seed(0)
    model = SequenceModel(ModelConfig(vocab_size=512, d_model=128, n_layers=3),
                          KLAConfig(d_state=16, backend="torch")).cuda().to(dtype).eval()
    ids = torch.randint(0, 512, (2, 24), generator=torch.Generator().manual_seed(2)).cuda()
    dec = kla_b200.ModelDecoder.from_model(model)
    tol = dict(rtol=1e-3, atol=1e-3) if dtype == torch.float32 else dict(rtol=5e-2, atol=1e-1)
    with torch.no_grad():
        ref_logits, ref_state = model(ids, state=model.init_state(2))
        logits, state = dec.prefill(ids)
        torch.testing.assert_close(logits.float(), ref_logits.float(), **tol)
        tok = ids[:, -1:]
        for _ in range(4):  # token-by-token, eagerly
            ref_l, ref_state = model(tok, state=ref_state)
            l = dec.step(tok[:, 0], state)
            torch.testing.assert_close(l.float(), ref_l[:, -1].float(), **tol)
            tok = ref_l[:, -1].argmax(-1, keepdim=True)
    if dtype == torch.float32:
        want = model.generate(ids, 12, temperature=0.0)
        lib = importlib.import_module("kalman-linear-attention_b200._lib").load()
        n0 = lib.kla_b200_launch_count()
        got = dec.generate(ids, 12)
        assert torch.equal(got, want), (got, want)
        assert torch.equal(dec.generate(ids, 12, use_graph=False), want)
        # prefill: conv + scan per layer; then two kernels per layer and token, captured once (+ two warm-up tokens)
        assert lib.kla_b200_launch_count() - n0 >= 3 * 2
