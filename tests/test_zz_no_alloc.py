"""The allocation-free forward entry point, ``kla_b200_scan_fwd_static``.

Some hosts of this library cannot ask for device memory: they run inside
another runtime's arena, or in a step where calling the allocator would
synchronise or could fail. For them the forward keeps its checkpoints in a
fixed buffer inside the library and hands back that buffer's address for the
backward. These tests call it through the C ABI, twice in a row with different
problems, and compare everything (forward outputs and the gradients of the
backward that reads the built-in buffer) with the ordinary entry point, whose
scratch the caller allocates.

Collected last on purpose (file name), so a stop-at-first-failure run has
already been through every other test.
"""

import ctypes
import importlib

import numpy as np
import pytest
import torch

L = importlib.import_module("kalman-linear-attention_b200._lib")


def _problem(B, T, M, S, seed, dev):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    d = dict(v=r(B, T, M), lambda_v=1.0 / torch.nn.functional.softplus(r(B, T, M)),
             k=r(B, T, S) * 0.3, q=r(B, T, S) * 0.3, a=torch.sigmoid(r(M, S)),
             p=torch.nn.functional.softplus(r(M, S)), dy=r(B, T, M), dyvar=r(B, T, M))
    return {n: t.to(dev).contiguous() for n, t in d.items()}


def _run(lib, d, B, T, M, S, static):
    dev = d["v"].device
    f32 = dict(device=dev, dtype=torch.float32)
    t3 = lambda t: L.Tensor3(t.data_ptr(), t.stride(0), t.stride(1))
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    out = {n: torch.empty(B, T, M, **f32) for n in ("y", "y_var", "dv", "dlambda_v")}
    out.update({n: torch.empty(B, M, S, **f32) for n in ("lam_fin", "eta_fin", "dlam0", "deta0")})
    out.update({n: torch.empty(B, T, S, **f32) for n in ("dk", "dq")})
    out.update({n: torch.empty(M, S, **f32) for n in ("da", "dp")})
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    fa = L.FwdArgs(B=B, L=T, M=M, S=S, in_dtype=0, out_dtype=0, decode_from_prior=0,
                   v=t3(d["v"]), lambda_v=t3(d["lambda_v"]), k=t3(d["k"]), q=t3(d["q"]),
                   a=P(d["a"]), p=P(d["p"]), lam0=None, eta0=None, y=t3(out["y"]), y_var=t3(out["y_var"]),
                   lam_fin=P(out["lam_fin"]), eta_fin=P(out["eta_fin"]), ckpt=None)
    if static:
        ck = ctypes.c_void_p()
        L.check(lib.kla_b200_scan_fwd_static(ctypes.byref(fa), stream, ctypes.byref(ck)))
        assert ck.value, "no scratch address returned"
        ckpt_ptr, keep = ck, None
    else:
        keep = torch.empty(lib.kla_b200_ckpt_bytes(B, T, M, S), device=dev, dtype=torch.uint8)
        fa.ckpt = keep.data_ptr()
        L.check(lib.kla_b200_scan_fwd(ctypes.byref(fa), stream))
        ckpt_ptr = P(keep)
    ba = L.BwdArgs(B=B, L=T, M=M, S=S, in_dtype=0, out_dtype=0, decode_from_prior=0,
                   v=t3(d["v"]), lambda_v=t3(d["lambda_v"]), k=t3(d["k"]), q=t3(d["q"]),
                   a=P(d["a"]), p=P(d["p"]), lam0=None, eta0=None, ckpt=ckpt_ptr,
                   dy=t3(d["dy"]), dy_var=t3(d["dyvar"]), dlam_fin=None, deta_fin=None,
                   dv=t3(out["dv"]), dlambda_v=t3(out["dlambda_v"]), dk=P(out["dk"]), dq=P(out["dq"]),
                   da=P(out["da"]), dp=P(out["dp"]), dlam0=P(out["dlam0"]), deta0=P(out["deta0"]))
    L.check(lib.kla_b200_scan_bwd(ctypes.byref(ba), stream))
    torch.cuda.synchronize(dev)
    return {n: t.cpu().numpy() for n, t in out.items()}


@pytest.mark.gpu
def test_static_scratch_forward_matches_ordinary_entry_point_twice():
    lib = L.load()
    dev = torch.device("cuda:0")
    # two different problems back to back: the second must not see the first's leftovers
    for (B, T, M, S), seed in (((2, 200, 96, 16), 0), ((3, 77, 40, 8), 1)):
        d = _problem(B, T, M, S, seed, dev)
        ref = _run(lib, d, B, T, M, S, static=False)
        got = _run(lib, d, B, T, M, S, static=True)
        for n in ref:
            assert np.isfinite(got[n]).all(), n
            if n in ("dk", "dq", "da", "dp"):  # atomically accumulated: order of adds varies
                np.testing.assert_allclose(got[n], ref[n], rtol=1e-4, atol=1e-5, err_msg=n)
            else:  # same kernels, same inputs: identical
                np.testing.assert_array_equal(got[n], ref[n], err_msg=n)
    assert L.device_status() == 0


@pytest.mark.gpu
def test_static_scratch_refuses_oversized_problems():
    lib = L.load()
    B, T, M, S = 8, 4096, 1024, 16  # 268 MB of checkpoints: far beyond the built-in buffer
    assert lib.kla_b200_ckpt_bytes(B, T, M, S) > L.STATIC_CKPT_BYTES
    before = lib.kla_b200_launch_count()
    ck = ctypes.c_void_p()
    fa = L.FwdArgs(B=B, L=T, M=M, S=S, in_dtype=0, out_dtype=0)
    rc = lib.kla_b200_scan_fwd_static(ctypes.byref(fa), None, ctypes.byref(ck))
    assert rc == 5 and not ck.value
    assert b"too large" in lib.kla_b200_strerror(rc)
    assert lib.kla_b200_launch_count() == before
    with pytest.raises(ValueError, match="too large"):
        L.check(rc)
