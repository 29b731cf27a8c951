"""ctypes view of ``libkla_b200.so``: the structs and prototypes of
``include/kla_b200.h``. Loading fails loudly when the library has not been
built; there is no fallback implementation."""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("KLA_B200_LIB") or os.path.join(HERE, "libkla_b200.so")

F32, BF16 = 0, 1
MAX_DSTATE = 128
STATIC_CKPT_BYTES = 32 << 20

SYMBOLS = (
    "kla_b200_ckpt_bytes",
    "kla_b200_segment_scratch_bytes",
    "kla_b200_plan_segments",
    "kla_b200_ckpt_interval",
    "kla_b200_scan_fwd",
    "kla_b200_scan_fwd_static",
    "kla_b200_scan_bwd",
    "kla_b200_step",
    "kla_b200_slab_aggregate",
    "kla_b200_chunk_fold",
    "kla_b200_epilogue_bwd",
    "kla_b200_conv_step",
    "kla_b200_conv_seq",
    "kla_b200_conv_seq_bwd",
    "kla_b200_step_layer",
    "kla_b200_mobius_scan_fwd",
    "kla_b200_mobius_scan_bwd",
    "kla_b200_affine_scan_fwd",
    "kla_b200_affine_scan_bwd",
    "kla_b200_strerror",
    "kla_b200_version",
    "kla_b200_launch_count",
    "kla_b200_device_status",
    "kla_b200_test_hooks",
)


class Tensor3(Structure):
    _fields_ = [("ptr", c_void_p), ("stride_b", c_int64), ("stride_t", c_int64)]


ACT = {"silu": 0, "gelu": 1, "relu": 2, None: 3}
MAX_CONV_TAPS = 8


class ConvStepArgs(Structure):
    _fields_ = [
        ("B", c_int64), ("D", c_int64), ("K", c_int64),
        ("dtype", c_int32), ("activation", c_int32),
        ("x", c_void_p), ("x_stride_b", c_int64),
        ("weight", c_void_p), ("bias", c_void_p), ("state", c_void_p), ("z", c_void_p),
    ]


class ConvSeqArgs(Structure):
    _fields_ = [
        ("B", c_int64), ("L", c_int64), ("D", c_int64), ("K", c_int64),
        ("dtype", c_int32), ("activation", c_int32),
        ("x", Tensor3), ("weight", c_void_p), ("bias", c_void_p), ("state", c_void_p), ("state_out", c_void_p),
        ("z", Tensor3),
    ]


class ConvSeqBwdArgs(Structure):
    _fields_ = [
        ("B", c_int64), ("L", c_int64), ("D", c_int64), ("K", c_int64),
        ("dtype", c_int32), ("activation", c_int32),
        ("x", Tensor3), ("dz", Tensor3), ("weight", c_void_p), ("bias", c_void_p), ("state", c_void_p),
        ("dx", Tensor3), ("dweight", c_void_p), ("dbias", c_void_p),
    ]


class StepLayerArgs(Structure):
    _fields_ = [
        ("B", c_int64), ("M", c_int64), ("S", c_int64),
        ("in_dtype", c_int32), ("out_dtype", c_int32), ("decode_from_prior", c_int32),
        ("qk_norm", c_int32), ("gate_activation", c_int32), ("lambda_skip_len", c_int32),
        ("obs_var_min", c_float), ("obs_var_max", c_float), ("clip_value", c_float),
        ("v", c_void_p), ("log_sigma_v", c_void_p), ("v_stride_b", c_int64), ("log_sigma_v_stride_b", c_int64),
        ("k", c_void_p), ("q", c_void_p), ("k_stride_b", c_int64), ("q_stride_b", c_int64),
        ("z", c_void_p), ("gate", c_void_p), ("z_stride_b", c_int64), ("gate_stride_b", c_int64),
        ("lambda_skip", c_void_p), ("a", c_void_p), ("p", c_void_p), ("lam", c_void_p), ("eta", c_void_p),
        ("y", c_void_p), ("y_var", c_void_p), ("lam_out", c_void_p), ("eta_out", c_void_p),
    ]


class RawScanArgs(Structure):
    _fields_ = [
        ("B", c_int64), ("L", c_int64), ("N", c_int64),
        ("inp", c_void_p * 6), ("out", c_void_p * 4),
        ("state0", c_void_p), ("dstate0", c_void_p),
    ]


class FwdArgs(Structure):
    _fields_ = [
        ("B", c_int64), ("L", c_int64), ("M", c_int64), ("S", c_int64),
        ("in_dtype", c_int32), ("out_dtype", c_int32), ("decode_from_prior", c_int32),
        ("v", Tensor3), ("lambda_v", Tensor3), ("k", Tensor3), ("q", Tensor3),
        ("a", c_void_p), ("p", c_void_p), ("lam0", c_void_p), ("eta0", c_void_p),
        ("y", Tensor3), ("y_var", Tensor3),
        ("lam_fin", c_void_p), ("eta_fin", c_void_p), ("ckpt", c_void_p),
        ("lambda_v_is_log_variance", c_int32), ("obs_var_min", c_float), ("obs_var_max", c_float),
        ("z", Tensor3), ("gate", Tensor3), ("lambda_skip", c_void_p),
        ("lambda_skip_len", c_int32), ("gate_activation", c_int32),
        ("y_raw", Tensor3), ("y_var_raw", Tensor3), ("work", c_void_p),
    ]


class EpilogueBwdArgs(Structure):
    _fields_ = [
        ("B", c_int64), ("L", c_int64), ("M", c_int64),
        ("in_dtype", c_int32), ("out_dtype", c_int32), ("gate_activation", c_int32), ("lambda_skip_len", c_int32),
        ("dout", Tensor3), ("dout_var", Tensor3), ("y_raw", Tensor3), ("y_var_raw", Tensor3),
        ("z", Tensor3), ("gate", Tensor3), ("lambda_skip", c_void_p),
        ("dy", Tensor3), ("dy_var", Tensor3), ("dz", Tensor3), ("dgate", Tensor3), ("dlambda_skip", c_void_p),
    ]


class BwdArgs(Structure):
    _fields_ = [
        ("B", c_int64), ("L", c_int64), ("M", c_int64), ("S", c_int64),
        ("in_dtype", c_int32), ("out_dtype", c_int32), ("decode_from_prior", c_int32),
        ("v", Tensor3), ("lambda_v", Tensor3), ("k", Tensor3), ("q", Tensor3),
        ("a", c_void_p), ("p", c_void_p), ("lam0", c_void_p), ("eta0", c_void_p),
        ("ckpt", c_void_p),
        ("dy", Tensor3), ("dy_var", Tensor3),
        ("dlam_fin", c_void_p), ("deta_fin", c_void_p),
        ("dv", Tensor3), ("dlambda_v", Tensor3),
        ("dk", c_void_p), ("dq", c_void_p), ("da", c_void_p), ("dp", c_void_p),
        ("dlam0", c_void_p), ("deta0", c_void_p),
        ("lambda_v_is_log_variance", c_int32), ("obs_var_min", c_float), ("obs_var_max", c_float),
    ]


class SlabArgs(Structure):
    _fields_ = [
        ("B", c_int64), ("L", c_int64), ("M", c_int64), ("S", c_int64),
        ("in_dtype", c_int32), ("out_dtype", c_int32), ("decode_from_prior", c_int32), ("adjoint", c_int32),
        ("v", Tensor3), ("lambda_v", Tensor3), ("k", Tensor3), ("q", Tensor3),
        ("a", c_void_p), ("p", c_void_p), ("lam0", c_void_p), ("eta0", c_void_p),
        ("dy", Tensor3), ("dy_var", Tensor3), ("out", c_void_p),
    ]


class ChunkFoldArgs(Structure):
    _fields_ = [
        ("B", c_int64), ("C", c_int64), ("M", c_int64), ("S", c_int64), ("adjoint", c_int32),
        ("agg", c_void_p), ("in_a", c_void_p), ("in_b", c_void_p), ("out_a", c_void_p), ("out_b", c_void_p),
    ]


class StepArgs(Structure):
    _fields_ = [
        ("B", c_int64), ("M", c_int64), ("S", c_int64),
        ("in_dtype", c_int32), ("out_dtype", c_int32), ("decode_from_prior", c_int32),
        ("v", c_void_p), ("lambda_v", c_void_p),
        ("v_stride_b", c_int64), ("lambda_v_stride_b", c_int64),
        ("k", c_void_p), ("q", c_void_p),
        ("k_stride_b", c_int64), ("q_stride_b", c_int64),
        ("a", c_void_p), ("p", c_void_p), ("lam", c_void_p), ("eta", c_void_p),
        ("y", c_void_p), ("y_var", c_void_p), ("lam_out", c_void_p), ("eta_out", c_void_p),
    ]


_lib = None


class LibraryMissing(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    """Load the library once; raise :class:`LibraryMissing` if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise LibraryMissing(
            f"{LIB_PATH} is not built. Build it with "
            "`python kalman-linear-attention_b200/build.py` (needs nvcc; no GPU needed to build). "
            "The b200 backend has no CPU or Triton fallback."
        )
    lib = ctypes.CDLL(LIB_PATH)
    lib.kla_b200_ckpt_bytes.restype = c_size_t
    lib.kla_b200_ckpt_bytes.argtypes = [c_int64] * 4
    lib.kla_b200_segment_scratch_bytes.restype = c_size_t
    lib.kla_b200_segment_scratch_bytes.argtypes = [c_int64] * 3
    lib.kla_b200_plan_segments.restype = c_int
    lib.kla_b200_plan_segments.argtypes = [c_int64, c_int64, c_int, c_int, c_int, POINTER(c_int)]
    lib.kla_b200_ckpt_interval.restype = c_int64
    lib.kla_b200_scan_fwd.restype = c_int
    lib.kla_b200_scan_fwd.argtypes = [POINTER(FwdArgs), c_void_p]
    lib.kla_b200_scan_fwd_static.restype = c_int
    lib.kla_b200_scan_fwd_static.argtypes = [POINTER(FwdArgs), c_void_p, POINTER(c_void_p)]
    lib.kla_b200_scan_bwd.restype = c_int
    lib.kla_b200_scan_bwd.argtypes = [POINTER(BwdArgs), c_void_p]
    lib.kla_b200_slab_aggregate.restype = c_int
    lib.kla_b200_slab_aggregate.argtypes = [POINTER(SlabArgs), c_void_p]
    lib.kla_b200_epilogue_bwd.restype = c_int
    lib.kla_b200_epilogue_bwd.argtypes = [POINTER(EpilogueBwdArgs), c_void_p]
    lib.kla_b200_chunk_fold.restype = c_int
    lib.kla_b200_chunk_fold.argtypes = [POINTER(ChunkFoldArgs), c_void_p]
    for name in ("mobius_scan_fwd", "mobius_scan_bwd", "affine_scan_fwd", "affine_scan_bwd"):
        fn = getattr(lib, "kla_b200_" + name)
        fn.restype = c_int
        fn.argtypes = [POINTER(RawScanArgs), c_void_p]
    lib.kla_b200_conv_step.restype = c_int
    lib.kla_b200_conv_step.argtypes = [POINTER(ConvStepArgs), c_void_p]
    lib.kla_b200_conv_seq.restype = c_int
    lib.kla_b200_conv_seq.argtypes = [POINTER(ConvSeqArgs), c_void_p]
    lib.kla_b200_conv_seq_bwd.restype = c_int
    lib.kla_b200_conv_seq_bwd.argtypes = [POINTER(ConvSeqBwdArgs), c_void_p]
    lib.kla_b200_step_layer.restype = c_int
    lib.kla_b200_step_layer.argtypes = [POINTER(StepLayerArgs), c_void_p]
    lib.kla_b200_step.restype = c_int
    lib.kla_b200_step.argtypes = [POINTER(StepArgs), c_void_p]
    lib.kla_b200_strerror.restype = c_char_p
    lib.kla_b200_strerror.argtypes = [c_int]
    lib.kla_b200_version.restype = c_int
    lib.kla_b200_launch_count.restype = c_int64
    lib.kla_b200_device_status.restype = c_int
    lib.kla_b200_device_status.argtypes = [POINTER(c_int)]
    lib.kla_b200_test_hooks.restype = c_int
    lib.kla_b200_test_hooks.argtypes = [c_int64, c_int32]
    _lib = lib
    return lib


def device_status() -> int:
    """Synchronise and return the device-side status word (0 = every kernel ran to
    its end; see ``kla_b200_device_status`` in ``include/kla_b200.h``)."""
    st = c_int(0)
    check(load().kla_b200_device_status(ctypes.byref(st)))
    return st.value


def check_status(what: str = "kla_b200") -> None:
    """Raise ``RuntimeError`` if a kernel launched so far on the current device gave up on a bounded wait
    (its outputs are then invalid). Synchronises, so call it where the caller synchronises anyway."""
    st = device_status()
    if st != 0:
        raise RuntimeError(f"{what}: a kernel gave up on a bounded wait (device status {st:#x}); its outputs are invalid")


def check(code: int) -> None:
    """Map a C-ABI status to the reference's exception convention:
    unsupported configuration -> NotImplementedError (src/kla/ops/cuda_backend.py:239-242),
    bad argument -> ValueError, CUDA failure -> RuntimeError."""
    if code == 0:
        return
    msg = load().kla_b200_strerror(code).decode()
    if code == 2:
        raise NotImplementedError(f"The b200 KLA backend: {msg}. Use backend='torch' for this case.")
    if code in (1, 4, 5):
        raise ValueError(f"kla_b200: {msg}")
    raise RuntimeError(f"kla_b200: {msg}")
