"""Layer decode (conv step + fused sensor/filter/gate step): the B200 kernels against the
reference layer's own token-by-token outputs (tests/golden/decode_*.npz)."""

import glob
import os
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import kla_b200  # noqa: E402
from conftest import reference_src  # noqa: E402
from importlib import import_module  # noqa: E402

decode = import_module("kalman-linear-attention_b200.decode")
CASES = sorted(os.path.basename(p)[7:-4] for p in glob.glob(os.path.join(HERE, "golden", "decode_*.npz")))
REF_SRC = reference_src()  # the directory holding the reference package `kla`, or "" when there is none here
needs_ref = pytest.mark.skipif(not os.path.isdir(REF_SRC), reason="reference package not present")


def load(name):
    z = dict(np.load(os.path.join(HERE, "golden", f"decode_{name}.npz")))
    weights = {k[2:]: torch.from_numpy(v) for k, v in z.items() if k.startswith("w:")}
    config = {}
    for k, v in z.items():
        if k.startswith("c:"):
            val = v.item()
            config[k[2:]] = None if val == "" else val
    return z, weights, config


def test_cases_present():
    assert CASES == ["bare", "default", "lowrank", "variant"]


@pytest.mark.parametrize("name", CASES)
def test_discretisation_matches_the_layer(name):
    z, weights, config = load(name)
    a_bar, p_bar = decode.discretize(weights, config)
    np.testing.assert_allclose(a_bar.numpy(), z["a_bar"], rtol=1e-6, atol=1e-8)
    np.testing.assert_allclose(p_bar.numpy(), z["p_bar"], rtol=1e-6, atol=1e-10)
    dec = kla_b200.LayerDecoder(weights, config)
    assert (dec.M, dec.S) == z["lam0"].shape[1:]
    assert dec.w_value + dec.w_var + 2 * dec.S == weights["sensor_proj.weight"].shape[0]


def test_cpu_tensors_are_refused():
    _, weights, config = load("default")
    dec = kla_b200.LayerDecoder(weights, config)
    with pytest.raises(NotImplementedError, match="CUDA"):
        dec.step(torch.zeros(2, 32), dec.init_state(2, "cpu"))
    with pytest.raises(ValueError, match="lacks"):
        kla_b200.LayerDecoder(weights, {"d_state": 8})


@needs_ref
def test_from_layer_reads_a_reference_layer():
    sys.path.insert(0, REF_SRC)
    try:
        import kla

        torch.manual_seed(0)
        layer = kla.KLALayer(32, kla.KLAConfig(d_state=8, lambda_skip_mode="vector"))
        dec = kla_b200.LayerDecoder.from_layer(layer)
        a_bar, p_bar = layer._compute_aq()
        torch.testing.assert_close(dec.a_bar, a_bar.detach())
        torch.testing.assert_close(dec.p_bar, p_bar.detach())
        assert dec.skip.shape == (layer.d_inner,) and dec.conv_w.shape == (layer.d_inner, 4)
    finally:
        sys.path.remove(REF_SRC)


# ----------------------------------------------------------------------- GPU

def _run(name, dtype, steps=3):
    dev = torch.device("cuda:0")
    z, weights, config = load(name)
    weights = {k: (v.to(dtype) if k.split(".")[0] in ("in_proj", "sensor_proj", "out_proj", "value_expand", "var_expand")
                   else v) for k, v in weights.items()}
    dec = kla_b200.LayerDecoder(weights, config).to(dev)
    conv = torch.from_numpy(z["conv0"]).to(dev, dtype) if "conv0" in z else None
    state = (conv, torch.from_numpy(z["lam0"]).to(dev), torch.from_numpy(z["eta0"]).to(dev))
    outs = []
    for t in range(steps):
        res = dec.step(torch.from_numpy(z["x"][t]).to(dev, dtype), state)
        outs.append(tuple(r.float().cpu() for r in (res if isinstance(res, tuple) else (res,))))
        outs[-1] += tuple(None if s is None else s.float().cpu().clone() for s in state)
    return z, config, outs


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_decode_matches_reference_layer_f32(name):
    z, config, outs = _run(name, torch.float32)
    for t, got in enumerate(outs):
        n_out = 2 if config["return_variance"] else 1
        torch.testing.assert_close(got[0], torch.from_numpy(z[f"out{t}"]), rtol=1e-4, atol=1e-5, msg=lambda m: f"out{t}: {m}")
        if n_out == 2:
            torch.testing.assert_close(got[1], torch.from_numpy(z[f"outvar{t}"]), rtol=1e-4, atol=1e-5)
        conv, lam, eta = got[n_out:]
        if conv is not None:
            torch.testing.assert_close(conv, torch.from_numpy(z[f"conv{t + 1}"]), rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(lam, torch.from_numpy(z[f"lam{t + 1}"]), rtol=2e-5, atol=1e-6)
        torch.testing.assert_close(eta, torch.from_numpy(z[f"eta{t + 1}"]), rtol=2e-5, atol=2e-6)
    L = import_module("kalman-linear-attention_b200._lib")
    assert L.device_status() == 0


@pytest.mark.gpu
def test_decode_bf16_activations_stay_close():
    z, config, outs = _run("default", torch.bfloat16)
    for t, got in enumerate(outs):
        ref = torch.from_numpy(z[f"out{t}"])
        assert (got[0] - ref).abs().max() <= 3e-2 * (1.0 + ref.abs().max())


@pytest.mark.gpu
def test_decode_step_is_graph_capturable():
    dev = torch.device("cuda:0")
    z, weights, config = load("default")
    dec = kla_b200.LayerDecoder(weights, config).to(dev)

    def fresh():
        return (torch.from_numpy(z["conv0"]).to(dev), torch.from_numpy(z["lam0"]).to(dev), torch.from_numpy(z["eta0"]).to(dev))

    x = torch.from_numpy(z["x"][0]).to(dev)
    state = fresh()
    dec.step(x, state)  # warm-up outside capture (library handles, lazy loads)
    state = fresh()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = dec.step(x, state)
    torch.cuda.current_stream().wait_stream(s)
    for buf, src in zip(state, fresh()):
        buf.copy_(src)
    g.replay()
    torch.cuda.synchronize()
    torch.testing.assert_close(out.cpu(), torch.from_numpy(z["out0"]), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(state[1].cpu(), torch.from_numpy(z["lam1"]), rtol=2e-5, atol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_prefill_then_decode_matches_reference_layer(name):
    """The whole inference route: prefill through the scan kernels (sensor prologue and skip/gate
    epilogue inside), then token-by-token decode from the state the prefill left."""
    dev = torch.device("cuda:0")
    z, weights, config = load(name)
    dec = kla_b200.LayerDecoder(weights, config).to(dev)
    pre, state = dec.prefill(torch.from_numpy(z["x0"]).to(dev))
    outs = pre if isinstance(pre, tuple) else (pre,)
    torch.testing.assert_close(outs[0].cpu(), torch.from_numpy(z["pre_out"]), rtol=1e-4, atol=2e-5)
    if config["return_variance"]:
        torch.testing.assert_close(outs[1].cpu(), torch.from_numpy(z["pre_outvar"]), rtol=1e-4, atol=2e-5)
    if "conv0" in z:
        torch.testing.assert_close(state[0].cpu(), torch.from_numpy(z["conv0"]), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(state[1].cpu(), torch.from_numpy(z["lam0"]), rtol=5e-5, atol=1e-5)
    torch.testing.assert_close(state[2].cpu(), torch.from_numpy(z["eta0"]), rtol=5e-5, atol=1e-5)
    for t in range(3):
        res = dec.step(torch.from_numpy(z["x"][t]).to(dev), state)
        out = res[0] if isinstance(res, tuple) else res
        torch.testing.assert_close(out.cpu(), torch.from_numpy(z[f"out{t}"]), rtol=2e-4, atol=3e-5)
    torch.testing.assert_close(state[1].cpu(), torch.from_numpy(z["lam3"]), rtol=1e-4, atol=1e-5)


# ------------------------------------------------------------ causal convolution over a sequence, forward + backward

def _conv_module_math(x, weight, bias, state, act):
    """CausalConv1d.forward (src/kla/layers/common.py:87-96) as plain torch operations."""
    B, L, D = x.shape
    K = weight.shape[-1]
    x_t = x.transpose(1, 2)
    if state is None:
        state = torch.zeros(B, D, K - 1, device=x.device, dtype=x.dtype)
    x_pad = torch.cat((state.to(x_t.dtype), x_t), dim=-1)
    y = torch.nn.functional.conv1d(x_pad, weight, bias, groups=D)
    return getattr(torch.nn.functional, act)(y).transpose(1, 2), x_pad[..., x_pad.shape[-1] - (K - 1):]


@pytest.mark.gpu
@pytest.mark.parametrize("B,L,D,K,act,with_state,with_bias", [
    (2, 200, 96, 4, "silu", False, True),     # the layer's defaults; L not a multiple of the kernels' chunks
    (1, 64, 130, 4, "gelu", True, True),      # carried window, channels not a multiple of the block
    (3, 129, 32, 8, "relu", True, False),     # most taps, no bias
    (2, 2, 16, 4, "silu", True, True),        # sequence shorter than the window
    (2, 33, 20, 1, "silu", False, True),      # one tap: no window at all
    (2, 70, 64, 2, "gelu", False, False),
])
def test_causal_conv_forward_backward(B, L, D, K, act, with_state, with_bias):
    layer = import_module("kalman-linear-attention_b200.layer")
    g = torch.Generator().manual_seed(B * 1000 + L + K)
    # x as the layer hands it over: one half of a wider projection, i.e. a view with a row stride of 2 D
    wide = torch.randn(B, L, 2 * D, generator=g).cuda()
    weight = (torch.randn(D, 1, K, generator=g) * 0.5).cuda().requires_grad_(True)
    bias = torch.randn(D, generator=g).cuda().requires_grad_(True) if with_bias else None
    state = torch.randn(B, D, K - 1, generator=g).cuda() if with_state else None
    dz = torch.randn(B, L, D, generator=g).cuda()

    def run(fn):
        w2 = wide.clone().requires_grad_(True)
        z, st = fn(w2[..., :D], weight, bias, state, act)
        grads = torch.autograd.grad(z, [w2, weight] + ([bias] if with_bias else []), dz)
        return [z.detach(), st.detach()] + [t.detach() for t in grads]

    got = run(layer.causal_conv_b200)
    want = run(_conv_module_math)
    names = ["z", "new_state", "dx", "dweight", "dbias"]
    for n, a_, b_ in zip(names, got, want):
        assert a_.shape == b_.shape, n
        torch.testing.assert_close(a_, b_, rtol=2e-5, atol=2e-5, msg=lambda m, n=n: f"{n}: {m}")


@pytest.mark.gpu
def test_causal_conv_bf16_tracks_float32():
    layer = import_module("kalman-linear-attention_b200.layer")
    g = torch.Generator().manual_seed(5)
    B, L, D, K = 2, 300, 256, 4
    x32 = torch.randn(B, L, D, generator=g).cuda()
    weight = (torch.randn(D, 1, K, generator=g) * 0.5).cuda().requires_grad_(True)
    bias = torch.randn(D, generator=g).cuda().requires_grad_(True)
    dz = torch.randn(B, L, D, generator=g).cuda()
    outs = {}
    for dt in (torch.float32, torch.bfloat16):
        x = x32.to(dt).requires_grad_(True)
        z, _ = layer.causal_conv_b200(x, weight, bias, None, "silu")
        assert z.dtype == dt
        outs[dt] = [z.float().detach()] + [t.float() for t in torch.autograd.grad(z, [x, weight, bias], dz.to(dt))]
    for a_, b_ in zip(outs[torch.bfloat16], outs[torch.float32]):
        assert ((a_ - b_).abs().max() / (b_.abs().max() + 1e-6)).item() < 2e-2
