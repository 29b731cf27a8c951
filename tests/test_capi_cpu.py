"""The C-ABI library without a GPU: it loads, exports every symbol the header
declares, and rejects bad arguments before touching CUDA."""

import ctypes
import importlib
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "kla_b200.h")


@pytest.fixture(scope="module")
def L():
    import kla_b200

    kla_b200.build()
    return importlib.import_module("kalman-linear-attention_b200._lib")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(kla_b200_\w+)\s*\(", text)))


def test_header_symbols_are_exported(L):
    lib = L.load()
    names = declared_functions()
    assert len(names) >= 8
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/kla_b200.h but not exported"
    assert set(L.SYMBOLS) <= set(names)


def test_version_and_checkpoint_size(L):
    lib = L.load()
    assert lib.kla_b200_version() >= 100
    iv = lib.kla_b200_ckpt_interval()
    assert iv == 8
    # one (P, mean) float2 per lane per started interval
    up = lambda n: (n + 255) // 256 * 256
    seg = lambda B, M, S: 2 * (256 + up(4 * B * M)) + up(8 * B * M * S) + up(20 * B * M * S)
    assert lib.kla_b200_segment_scratch_bytes(8, 1024, 16) == seg(8, 1024, 16)
    assert lib.kla_b200_ckpt_bytes(8, 4096, 1024, 16) == up(8 * (4096 // iv) * 1024 * 16 * 8) + seg(8, 1024, 16)
    assert lib.kla_b200_ckpt_bytes(2, 17, 3, 5) == up(2 * 3 * 3 * 5 * 8) + seg(2, 3, 5)
    assert lib.kla_b200_ckpt_bytes(0, 17, 3, 5) == 0


def test_bad_arguments_are_rejected_without_cuda(L):
    lib = L.load()
    assert lib.kla_b200_scan_fwd(None, None) == 1
    assert lib.kla_b200_scan_bwd(None, None) == 1
    assert lib.kla_b200_step(None, None) == 1
    a = L.FwdArgs(B=1, L=4, M=2, S=200, in_dtype=0, out_dtype=0)
    assert lib.kla_b200_scan_fwd(ctypes.byref(a), None) == 2  # d_state above the cap
    a = L.FwdArgs(B=1, L=4, M=2, S=4, in_dtype=7, out_dtype=0)
    assert lib.kla_b200_scan_fwd(ctypes.byref(a), None) == 2  # unknown dtype
    a = L.FwdArgs(B=1, L=4, M=2, S=4, in_dtype=0, out_dtype=1)
    assert lib.kla_b200_scan_fwd(ctypes.byref(a), None) == 2  # f32 in, bf16 out is not a pair
    a = L.FwdArgs(B=-1, L=4, M=2, S=4)
    assert lib.kla_b200_scan_fwd(ctypes.byref(a), None) == 1
    a = L.FwdArgs(B=1, L=4, M=2, S=4)  # all pointers NULL
    assert lib.kla_b200_scan_fwd(ctypes.byref(a), None) == 1
    # empty problems are fine and launch nothing
    a = L.FwdArgs(B=0, L=4, M=2, S=4)
    assert lib.kla_b200_scan_fwd(ctypes.byref(a), None) == 0
    assert lib.kla_b200_launch_count() == 0


def test_new_entry_points_reject_bad_arguments_without_cuda(L):
    lib = L.load()
    for name in ("mobius_scan_fwd", "mobius_scan_bwd", "affine_scan_fwd", "affine_scan_bwd"):
        fn = getattr(lib, "kla_b200_" + name)
        assert fn(None, None) == 1
        assert fn(ctypes.byref(L.RawScanArgs(B=1, L=4, N=8)), None) == 1       # NULL tensors
        assert fn(ctypes.byref(L.RawScanArgs(B=-1, L=4, N=8)), None) == 1
        assert fn(ctypes.byref(L.RawScanArgs(B=1 << 20, L=4, N=8)), None) == 2  # batch above the grid limit
    buf = (ctypes.c_float * 64)()
    a = L.RawScanArgs(B=1, L=4, N=8, state0=ctypes.addressof(buf))
    assert lib.kla_b200_affine_scan_fwd(ctypes.byref(a), None) == 1            # the affine scan takes no initial state
    a = L.RawScanArgs(B=1, L=4, N=8)
    for i in range(2):
        a.inp[i] = ctypes.addressof(buf) + 2                                   # not aligned to a float
    a.out[0] = ctypes.addressof(buf)
    assert lib.kla_b200_affine_scan_fwd(ctypes.byref(a), None) == 4

    assert lib.kla_b200_conv_step(None, None) == 1
    assert lib.kla_b200_conv_step(ctypes.byref(L.ConvStepArgs(B=1, D=4, K=9)), None) == 2   # more taps than supported
    assert lib.kla_b200_conv_step(ctypes.byref(L.ConvStepArgs(B=1, D=4, K=4, dtype=5)), None) == 2
    assert lib.kla_b200_conv_step(ctypes.byref(L.ConvStepArgs(B=1, D=4, K=4, activation=9)), None) == 1
    assert lib.kla_b200_conv_step(ctypes.byref(L.ConvStepArgs(B=1, D=4, K=4)), None) == 1   # NULL tensors
    assert lib.kla_b200_conv_step(ctypes.byref(L.ConvStepArgs(B=0, D=4, K=4)), None) == 0

    assert lib.kla_b200_conv_seq(None, None) == 1
    assert lib.kla_b200_conv_seq(ctypes.byref(L.ConvSeqArgs(B=1, L=8, D=4, K=9)), None) == 2
    assert lib.kla_b200_conv_seq(ctypes.byref(L.ConvSeqArgs(B=1, L=8, D=4, K=4)), None) == 1   # NULL tensors
    buf = (ctypes.c_float * 64)()
    same = L.ConvSeqArgs(B=1, L=8, D=4, K=4, weight=ctypes.addressof(buf), state=ctypes.addressof(buf),
                         state_out=ctypes.addressof(buf))
    assert lib.kla_b200_conv_seq(ctypes.byref(same), None) == 1                                # state_out aliases state
    assert lib.kla_b200_conv_seq(ctypes.byref(L.ConvSeqArgs(B=1, L=0, D=4, K=4)), None) == 0
    assert lib.kla_b200_conv_seq_bwd(None, None) == 1
    assert lib.kla_b200_conv_seq_bwd(ctypes.byref(L.ConvSeqBwdArgs(B=1, L=8, D=4, K=9)), None) == 2
    assert lib.kla_b200_conv_seq_bwd(ctypes.byref(L.ConvSeqBwdArgs(B=1, L=8, D=4, K=4, activation=9)), None) == 1
    assert lib.kla_b200_conv_seq_bwd(ctypes.byref(L.ConvSeqBwdArgs(B=1, L=8, D=4, K=4)), None) == 1   # NULL tensors
    assert lib.kla_b200_conv_seq_bwd(ctypes.byref(L.ConvSeqBwdArgs(B=1, L=8, D=4, K=4, weight=ctypes.addressof(buf))),
                                     None) == 1                                                        # no dweight
    assert lib.kla_b200_conv_seq_bwd(ctypes.byref(L.ConvSeqBwdArgs(B=1, L=0, D=4, K=4)), None) == 0
    assert lib.kla_b200_step_layer(None, None) == 1
    assert lib.kla_b200_step_layer(ctypes.byref(L.StepLayerArgs(B=1, M=4, S=200)), None) == 2
    assert lib.kla_b200_step_layer(ctypes.byref(L.StepLayerArgs(B=1, M=4, S=4, gate_activation=7)), None) == 1
    assert lib.kla_b200_step_layer(ctypes.byref(L.StepLayerArgs(B=1, M=4, S=4, lambda_skip_len=3)), None) == 1
    assert lib.kla_b200_step_layer(ctypes.byref(L.StepLayerArgs(B=1, M=4, S=4)), None) == 1  # NULL tensors
    assert lib.kla_b200_launch_count() == 0


def test_sizes_that_overflow_are_refused_not_wrapped(L):
    lib = L.load()
    size_max = ctypes.c_size_t(-1).value
    # 2^66 bytes: the product must saturate, not wrap to a small number
    assert lib.kla_b200_ckpt_bytes(1, 1 << 30, 1 << 30, 128) == size_max
    assert lib.kla_b200_ckpt_bytes(65535, 1 << 30, 1 << 30, 128) == size_max
    buf = (ctypes.c_float * 64)()
    ptr = ctypes.addressof(buf)
    a = L.FwdArgs(B=1, L=1 << 30, M=1 << 30, S=128)
    out = ctypes.c_void_p()
    assert lib.kla_b200_scan_fwd_static(ctypes.byref(a), None, ctypes.byref(out)) == 5  # too big for the built-in scratch
    assert out.value is None
    # a decode step whose grid would not fit 31 bits is refused instead of running a truncated grid
    big = dict(B=65535, M=1 << 30, S=128, in_dtype=0, out_dtype=0)
    s_args = L.StepArgs(v=ptr, lambda_v=ptr, k=ptr, q=ptr, a=ptr, p=ptr, lam=ptr, eta=ptr, y=ptr, y_var=ptr,
                        lam_out=ptr, eta_out=ptr, **big)
    assert lib.kla_b200_step(ctypes.byref(s_args), None) == 2
    l_args = L.StepLayerArgs(v=ptr, log_sigma_v=ptr, k=ptr, q=ptr, a=ptr, p=ptr, lam=ptr, eta=ptr, y=ptr, y_var=ptr,
                             lam_out=ptr, eta_out=ptr, **big)
    assert lib.kla_b200_step_layer(ctypes.byref(l_args), None) == 2
    assert lib.kla_b200_test_hooks(-1, 0) == 1
    assert lib.kla_b200_test_hooks(0, -1) == 0
    assert lib.kla_b200_launch_count() == 0


def test_error_text_and_exception_mapping(L):
    lib = L.load()
    assert lib.kla_b200_strerror(0) == b"ok"
    assert b"invalid" in lib.kla_b200_strerror(1)
    with pytest.raises(NotImplementedError, match="backend='torch'"):
        L.check(2)
    with pytest.raises(ValueError):
        L.check(1)
    with pytest.raises(ValueError):
        L.check(4)


def test_missing_library_fails_loudly(L, monkeypatch):
    monkeypatch.setattr(L, "_lib", None)
    monkeypatch.setattr(L, "LIB_PATH", "/nonexistent/libkla_b200.so")
    with pytest.raises(L.LibraryMissing, match="no CPU or Triton fallback"):
        L.load()


def test_segment_plan(L):
    """Host logic of the segmented kernels: when sequences are cut, into how many segments of what length."""
    lib = L.load()

    def plan(seqs, steps, backward, sms=148, forced=-1):
        n = ctypes.c_int(0)
        return lib.kla_b200_plan_segments(seqs, steps, int(backward), sms, forced, ctypes.byref(n)), n.value

    assert plan(128, 4096, True) == (1, 4096)            # no more sequences than SMs: every CTA has an SM to itself
    assert plan(256, 4096, True) == (16, 256)            # up to two per SM: the backward in 16 segments
    assert plan(256, 4096, False) == (1, 4096)           # the forward only from two sequences per SM on
    assert plan(320, 4096, True) == (8, 512) and plan(320, 4096, False) == (8, 512)
    assert plan(768, 2048, True) == (8, 256)
    assert plan(512, 256, True) == (1, 256)              # too short to cut (segments of at least 256 steps)
    assert plan(512, 600, True) == (3, 256)              # ragged last segment: 256 + 256 + 88
    assert plan(320, 4096, True, forced=0) == (1, 4096)
    assert plan(4, 100, True, forced=4) == (4, 32)       # forced: whole tiles of 16 steps
    assert plan(4, 16, True, forced=4) == (1, 16)
    n, length = plan(320, 1 << 20, True)
    assert n == 8 and length % 16 == 0 and n * length >= 1 << 20
