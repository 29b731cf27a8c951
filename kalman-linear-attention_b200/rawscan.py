"""The raw scan pair over materialised coefficients, on the B200 kernels.

Mirrors the reference's ``tiled_mobius_scan(A, B, C, D, lam0=None)`` and
``tiled_affine_scan(alpha, r)`` (src/kla/ops/kernels/triton/tiled_mobius_scan.py:301-311):
differentiable, float32, every tensor ``[B, L, M, S]``, ``lam0`` ``[B, M, S]``.

    lam_t = (A_t lam_{t-1} + B_t) / (C_t lam_{t-1} + D_t),  lam_{-1} = lam0 (ones when None)
    eta_t = alpha_t eta_{t-1} + r_t,                        eta_{-1} = 0

The backwards are the reference's exact adjoints (``TiledMobiusScan.backward``, :266-279;
``TiledAffineScan.backward``, :289-296) as one reverse-time kernel each. There is no CPU,
Triton or eager path: a tensor that is not a CUDA float32 tensor raises ``NotImplementedError``.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib


def _require(name: str, t: torch.Tensor) -> None:
    if not t.is_cuda:
        raise NotImplementedError(
            f"The b200 raw scans need CUDA tensors; {name} is on {t.device}. "
            "Use the reference's torch path (kla_scan(..., backend='torch')) on this device."
        )
    if t.dtype != torch.float32:
        raise NotImplementedError(
            f"The b200 raw scans run in float32 (like the reference's tiled scans); {name} is {t.dtype}. "
            "Use backend='torch' for other precisions."
        )


def _launch(name: str, shape, ins, outs, state0=None, dstate0=None) -> None:
    B, L, M, S = shape
    args = _lib.RawScanArgs(B=B, L=L, N=M * S)
    for i, t in enumerate(ins):
        args.inp[i] = t.data_ptr()
    for i, t in enumerate(outs):
        args.out[i] = t.data_ptr()
    args.state0 = state0.data_ptr() if state0 is not None else None
    args.dstate0 = dstate0.data_ptr() if dstate0 is not None else None
    lib = _lib.load()
    with torch.cuda.device(ins[0].device):
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        _lib.check(getattr(lib, "kla_b200_" + name)(ctypes.byref(args), stream))


class _MobiusScanB200(torch.autograd.Function):
    @staticmethod
    def forward(ctx, A, B, C, D, lam0):
        A, B, C, D = (t.contiguous() for t in (A, B, C, D))
        lam0c = lam0.contiguous() if lam0 is not None else None
        lam = torch.empty_like(A)
        _launch("mobius_scan_fwd", A.shape, (A, B, C, D), (lam,), state0=lam0c)
        ctx.save_for_backward(A, B, C, D, lam, *((lam0c,) if lam0c is not None else ()))
        ctx.has_lam0 = lam0c is not None
        return lam

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dlam):
        A, B, C, D, lam, *rest = ctx.saved_tensors
        lam0 = rest[0] if ctx.has_lam0 else None
        dlam = dlam.contiguous()
        dA, dB, dC, dD = (torch.empty_like(A) for _ in range(4))
        dlam0 = torch.empty_like(lam0) if (lam0 is not None and ctx.needs_input_grad[4]) else None
        _launch("mobius_scan_bwd", A.shape, (A, B, C, D, lam, dlam), (dA, dB, dC, dD), state0=lam0, dstate0=dlam0)
        return dA, dB, dC, dD, dlam0


class _AffineScanB200(torch.autograd.Function):
    @staticmethod
    def forward(ctx, alpha, r):
        alpha, r = alpha.contiguous(), r.contiguous()
        eta = torch.empty_like(alpha)
        _launch("affine_scan_fwd", alpha.shape, (alpha, r), (eta,))
        ctx.save_for_backward(alpha, eta)
        return eta

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, deta):
        alpha, eta = ctx.saved_tensors
        deta = deta.contiguous()
        dalpha, dr = torch.empty_like(alpha), torch.empty_like(alpha)
        _launch("affine_scan_bwd", alpha.shape, (alpha, eta, deta), (dalpha, dr))
        return dalpha, dr


def _check_shapes(first: torch.Tensor, others, names) -> None:
    if first.dim() != 4:
        raise ValueError(f"expected [B, L, M, S] coefficients, got shape {tuple(first.shape)}")
    for name, t in zip(names, others):
        if t.shape != first.shape:
            raise ValueError(f"{name} has shape {tuple(t.shape)}, expected {tuple(first.shape)}")


def mobius_scan_b200(A, B, C, D, lam0=None):
    """Differentiable Moebius scan -> ``lam`` ``[B, L, M, S]`` (reference: ``tiled_mobius_scan``)."""
    for name, t in (("A", A), ("B", B), ("C", C), ("D", D)):
        _require(name, t)
    _check_shapes(A, (B, C, D), ("B", "C", "D"))
    if A.numel() == 0:
        return torch.empty_like(A)
    if lam0 is not None:
        _require("lam0", lam0)
        if tuple(lam0.shape) != (A.shape[0], A.shape[2], A.shape[3]):
            raise ValueError(f"lam0 has shape {tuple(lam0.shape)}, expected [B, M, S]")
    return _MobiusScanB200.apply(A, B, C, D, lam0)


def affine_scan_b200(alpha, r):
    """Differentiable affine scan -> ``eta`` ``[B, L, M, S]`` (reference: ``tiled_affine_scan``)."""
    _require("alpha", alpha)
    _require("r", r)
    _check_shapes(alpha, (r,), ("r",))
    if alpha.numel() == 0:
        return torch.empty_like(alpha)
    return _AffineScanB200.apply(alpha, r)
