"""Host side of the ``b200`` backend: the reference's backend-callable contract
over the C-ABI library.

The reference dispatches ``kla_scan(..., backend=name)`` to a callable

    fn(v, lambda_v, k, q, a, p, initial_state=None, decode_from_prior=False)
        -> (y [B,L,M], y_var [B,L,M], KLAState(lam, eta) [B,M,S])

looked up in ``kla.ops.kla_ops._BACKENDS`` (src/kla/ops/kla_ops.py:430-442,
486-541). :func:`kla_scan_b200` is such a callable; :func:`kla_step_b200`
mirrors ``kla_step`` (src/kla/ops/kla_ops.py:293-331). Error behaviour follows
the reference's GPU backends (src/kla/ops/cuda_backend.py:239-275): a request
the kernels cannot serve raises ``NotImplementedError`` naming a backend that
can; nothing falls back silently, and there is no CPU or Triton path.
"""

from __future__ import annotations

import contextlib
import ctypes
import sys
from typing import NamedTuple, Optional

import torch

from . import _lib
from ._lib import BF16, F32, MAX_DSTATE, BwdArgs, ChunkFoldArgs, EpilogueBwdArgs, FwdArgs, SlabArgs, StepArgs, Tensor3


class KLAState(NamedTuple):
    """Filter state: posterior precision and information vector, each [B, M, S]
    (same fields as the reference's ``KLAState``, src/kla/ops/kla_ops.py:47-51)."""

    lam: torch.Tensor
    eta: torch.Tensor


def init_state(batch: int, d_model: int, d_state: int, device=None, dtype=torch.float32) -> KLAState:
    """Unit prior: precision 1, zero mean (src/kla/ops/kla_ops.py:54-61)."""
    return KLAState(
        lam=torch.ones(batch, d_model, d_state, device=device, dtype=dtype),
        eta=torch.zeros(batch, d_model, d_state, device=device, dtype=dtype),
    )


def _state_cls():
    """The reference's own KLAState when the reference package is loaded, so
    that callers doing isinstance checks or tuple unpacking see what they expect."""
    mod = sys.modules.get("kla.ops.kla_ops")
    return getattr(mod, "KLAState", KLAState) if mod is not None else KLAState


def _unsupported(msg: str) -> NotImplementedError:
    return NotImplementedError(
        f"The b200 KLA backend {msg}. Use backend='torch' (any device) or 'triton' for this case."
    )


_SM100_CACHE: dict = {}


def _require_device(t: torch.Tensor) -> None:
    """The kernels exist for CUDA tensors on an sm_100 device only."""
    if not t.is_cuda:
        raise _unsupported("requires CUDA tensors")
    _require_sm100(t.device)


def _require_sm100(device: torch.device) -> None:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    ok = _SM100_CACHE.get(idx)
    if ok is None:
        ok = torch.cuda.get_device_capability(idx)[0] == 10
        _SM100_CACHE[idx] = ok
    if not ok:
        raise _unsupported("is compiled for sm_100a (B200) only and this device is not one")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _t3(t: Optional[torch.Tensor]) -> Tensor3:
    if t is None:
        return Tensor3(None, 0, 0)
    return Tensor3(t.data_ptr(), t.stride(0), t.stride(1))


def _rowmajor_last(t: torch.Tensor) -> torch.Tensor:
    """The kernels take a batch and a time stride per tensor but need unit stride
    on the last dimension; anything else is copied once."""
    if t.dim() == 3 and (t.shape[-1] <= 1 or t.stride(-1) == 1):
        return t
    return t.contiguous()


_NULL_CTX = contextlib.nullcontext()


def _on(device: torch.device):
    """Context that makes ``device`` current for a launch; free when it already is (the usual case)."""
    idx = device.index
    if idx is None or idx == torch.cuda.current_device():
        return _NULL_CTX
    return torch.cuda.device(device)


def _stream(device: torch.device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _dt(t: torch.dtype) -> int:
    return BF16 if t == torch.bfloat16 else F32


def _sensor_fields(sensors):
    """C-ABI fields of the fused sensor prologue: ``sensors`` is None or (obs_var_min, obs_var_max or None)."""
    if sensors is None:
        return dict(lambda_v_is_log_variance=0, obs_var_min=0.0, obs_var_max=0.0)
    return dict(lambda_v_is_log_variance=1, obs_var_min=float(sensors[0]), obs_var_max=float(sensors[1] or 0.0))


def _epilogue_fields(epilogue):
    """C-ABI fields of the forward-only layer epilogue: ``epilogue`` is None or a dict with any of
    ``z`` + ``lambda_skip`` (float32, one value or [M]) and ``gate`` + ``gate_activation``."""
    if not epilogue:
        return {}
    out = {}
    skip = epilogue.get("lambda_skip")
    if skip is not None:
        out.update(z=_t3(epilogue["z"]), lambda_skip=_ptr(skip), lambda_skip_len=skip.numel())
    if epilogue.get("gate") is not None:
        out.update(gate=_t3(epilogue["gate"]), gate_activation=_lib.ACT[epilogue.get("gate_activation", "silu")])
    return out


_SM_COUNT: dict = {}


def _forward_segments(lib, dev: torch.device, B: int, L: int, M: int, S: int) -> bool:
    """Whether the forward kernel would cut a problem of this shape into segments (``kla_b200_plan_segments``)."""
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    lpc = 1
    while 4 * lpc < S:
        lpc *= 2
    per_cta = 128 // lpc  # channels per CTA of the scan kernels
    return lib.kla_b200_plan_segments(B * ((M + per_cta - 1) // per_cta), L, 0, _SM_COUNT[idx], -1, None) > 1


def _launch_fwd(v, lambda_v, k, q, a, p, lam0, eta0, prior: bool, out_dtype, need_ckpt: bool, sensors=None,
                epilogue=None, raw=None):
    """Allocate outputs (and the checkpoint scratch when a backward will follow)
    and enqueue ``kla_b200_scan_fwd`` on the current stream of the inputs' device."""
    lib = _lib.load()
    B, L, M = v.shape
    S = k.shape[2]
    dev = v.device
    y = torch.empty((B, L, M), device=dev, dtype=out_dtype)
    y_var = torch.empty((B, L, M), device=dev, dtype=out_dtype)
    lam_fin = torch.empty((B, M, S), device=dev, dtype=torch.float32)
    eta_fin = torch.empty((B, M, S), device=dev, dtype=torch.float32)
    ckpt = work = None
    if need_ckpt and L > 0:
        ckpt = torch.empty(lib.kla_b200_ckpt_bytes(B, L, M, S), device=dev, dtype=torch.uint8)
    elif _forward_segments(lib, dev, B, L, M, S):
        # no backward will follow, but the sequences are many enough for the kernel to hand them from CTA to CTA in
        # segments: that needs a little working memory
        work = torch.empty(lib.kla_b200_segment_scratch_bytes(B, M, S), device=dev, dtype=torch.uint8)
    args = FwdArgs(
        B=B, L=L, M=M, S=S, in_dtype=_dt(v.dtype), out_dtype=_dt(out_dtype),
        decode_from_prior=int(prior),
        v=_t3(v), lambda_v=_t3(lambda_v), k=_t3(k), q=_t3(q),
        a=_ptr(a), p=_ptr(p), lam0=_ptr(lam0), eta0=_ptr(eta0),
        y=_t3(y), y_var=_t3(y_var), lam_fin=_ptr(lam_fin), eta_fin=_ptr(eta_fin),
        ckpt=_ptr(ckpt), work=_ptr(work), **_sensor_fields(sensors), **_epilogue_fields(epilogue),
        **({} if raw is None else dict(y_raw=_t3(raw[0]), y_var_raw=_t3(raw[1]))),
    )
    with _on(dev):
        _lib.check(lib.kla_b200_scan_fwd(ctypes.byref(args), _stream(dev)))
    return y, y_var, lam_fin, eta_fin, ckpt


def _launch_bwd(v, lambda_v, k, q, a, p, lam0, eta0, ckpt, dy, dy_var, dlam_fin, deta_fin,
                prior: bool, out_dtype, sensors=None):
    """Allocate the gradients and enqueue ``kla_b200_scan_bwd``."""
    lib = _lib.load()
    B, L, M = v.shape
    S = k.shape[2]
    dev = v.device
    dv = torch.empty((B, L, M), device=dev, dtype=v.dtype)
    dlv = torch.empty((B, L, M), device=dev, dtype=v.dtype)
    dk = torch.empty((B, L, S), device=dev, dtype=torch.float32)
    dq = torch.empty((B, L, S), device=dev, dtype=torch.float32)
    da = torch.empty((M, S), device=dev, dtype=torch.float32)
    dp = torch.empty((M, S), device=dev, dtype=torch.float32)
    dlam0 = torch.empty((B, M, S), device=dev, dtype=torch.float32)
    deta0 = torch.empty((B, M, S), device=dev, dtype=torch.float32)
    args = BwdArgs(
        B=B, L=L, M=M, S=S, in_dtype=_dt(v.dtype), out_dtype=_dt(out_dtype),
        decode_from_prior=int(prior),
        v=_t3(v), lambda_v=_t3(lambda_v), k=_t3(k), q=_t3(q),
        a=_ptr(a), p=_ptr(p), lam0=_ptr(lam0), eta0=_ptr(eta0), ckpt=_ptr(ckpt),
        dy=_t3(dy), dy_var=_t3(dy_var), dlam_fin=_ptr(dlam_fin), deta_fin=_ptr(deta_fin),
        dv=_t3(dv), dlambda_v=_t3(dlv), dk=_ptr(dk), dq=_ptr(dq), da=_ptr(da), dp=_ptr(dp),
        dlam0=_ptr(dlam0), deta0=_ptr(deta0), **_sensor_fields(sensors),
    )
    with _on(dev):
        _lib.check(lib.kla_b200_scan_bwd(ctypes.byref(args), _stream(dev)))
    return dv, dlv, dk, dq, da, dp, dlam0, deta0


def slab_aggregate(v, lambda_v, k, a, p, *, q=None, dy=None, dy_var=None, lam0=None, eta0=None,
                   prior: bool = False) -> torch.Tensor:
    """Launch ``kla_b200_slab_aggregate``: one record per lane that describes how a whole time slab acts on
    the filter state (``dy`` None) or on the backward carry (``dy`` given). Returns [B, M, S, 8] float32."""
    lib = _lib.load()
    B, L, M = v.shape
    S = k.shape[2]
    out = torch.empty((B, M, S, 8), device=v.device, dtype=torch.float32)
    adjoint = dy is not None
    od = dy.dtype if adjoint else torch.float32
    args = SlabArgs(
        B=B, L=L, M=M, S=S, in_dtype=_dt(v.dtype), out_dtype=_dt(od),
        decode_from_prior=int(prior), adjoint=int(adjoint),
        v=_t3(v), lambda_v=_t3(lambda_v), k=_t3(k), q=_t3(q),
        a=_ptr(a), p=_ptr(p), lam0=_ptr(lam0), eta0=_ptr(eta0),
        dy=_t3(dy), dy_var=_t3(dy_var), out=_ptr(out),
    )
    with _on(v.device):
        _lib.check(lib.kla_b200_slab_aggregate(ctypes.byref(args), _stream(v.device)))
    return out


def chunk_fold(agg: torch.Tensor, C: int, in_a, in_b, adjoint: bool):
    """Launch ``kla_b200_chunk_fold`` over aggregates [B*C, M, S, 8]; returns two [B*C, M, S] float32 tensors:
    the state before each chunk (forward) or the state-gradient seeds of each chunk (adjoint)."""
    lib = _lib.load()
    BC, M, S, _ = agg.shape
    out_a = torch.empty((BC, M, S), device=agg.device, dtype=torch.float32)
    out_b = torch.empty((BC, M, S), device=agg.device, dtype=torch.float32)
    args = ChunkFoldArgs(B=BC // C, C=C, M=M, S=S, adjoint=int(adjoint), agg=_ptr(agg),
                         in_a=_ptr(in_a), in_b=_ptr(in_b), out_a=_ptr(out_a), out_b=_ptr(out_b))
    with _on(agg.device):
        _lib.check(lib.kla_b200_chunk_fold(ctypes.byref(args), _stream(agg.device)))
    return out_a, out_b


# CTAs the backward kernel keeps resident on a B200: 148 SMs x 2
_RESIDENT_CTAS = 296
_MIN_CHUNK_STEPS = 64


def _chunkable(t: Optional[torch.Tensor], B: int, L: int) -> bool:
    """[B, L, X] can be read as [B*C, L/C, X] without a copy."""
    return t is None or B == 1 or t.stride(0) == L * t.stride(1)


def pick_time_chunks(B: int, L: int, M: int, S: int, requested: Optional[int] = None) -> int:
    """Number of time chunks for the time-parallel scan. 1 = the plain lane-serial kernels.

    The kernels put one CTA on every 32 / 16 / 8 ... channels (d_state 16 / 32 / 64 ...) of every batch element.
    When that grid leaves most of the GPU empty, the sequence is cut into C chunks that run as B*C batch entries;
    building the chunks' start states costs about 0.7x of a forward + backward pass on top, so chunking is only
    chosen when the plain grid fills less than a third of the resident CTA slots; then up to 16 chunks, enough
    for about four waves of CTAs. C divides L, chunks keep at least 64 steps. ``requested`` (or the environment variable KLA_B200_TIME_CHUNKS) overrides the choice; it is
    lowered to the nearest usable divisor of L."""
    import os

    if requested is None and os.environ.get("KLA_B200_TIME_CHUNKS"):
        requested = int(os.environ["KLA_B200_TIME_CHUNKS"])
    lpc = 1
    while 4 * lpc < S:
        lpc *= 2
    mc = 4 * (32 // lpc)
    ctas = B * ((M + mc - 1) // mc)
    if requested is None:
        if ctas == 0 or 3 * ctas > _RESIDENT_CTAS:
            return 1
        # measured on B200 (T=4096, M=1024): several waves of short chunks beat one wave of long ones, up to 16 chunks
        want = min(16, (4 * _RESIDENT_CTAS) // ctas)
    else:
        want = max(1, int(requested))
    want = min(want, max(1, L // _MIN_CHUNK_STEPS), max(1, 65535 // max(B, 1)))
    for c in range(want, 0, -1):
        if L % c == 0:
            return c
    return 1


def _as_chunks(t: Optional[torch.Tensor], C: int) -> Optional[torch.Tensor]:
    """View [B, L, X] as [B*C, L/C, X] (same memory)."""
    if t is None or C == 1:
        return t
    B, L, X = t.shape
    if B == 1:
        return t.as_strided((C, L // C, X), (t.stride(1) * (L // C), t.stride(1), t.stride(2)), t.storage_offset())
    return t.as_strided((B * C, L // C, X), (t.stride(1) * (L // C), t.stride(1), t.stride(2)), t.storage_offset())


class _KLAScanB200(torch.autograd.Function):
    """Forward and exact backward of the fused scan, both as single kernels.

    Inputs are already canonical: v, lambda_v, k, q share one dtype (float32 or
    bfloat16) with unit last stride; a, p float32 contiguous [M, S]; lam0/eta0
    float32 contiguous [B, M, S] or None."""

    @staticmethod
    def forward(ctx, v, lambda_v, k, q, a, p, lam0, eta0, prior: bool, out_dtype: torch.dtype, sensors=None,
                chunks: int = 1):
        need_grad = any(ctx.needs_input_grad[:8])
        B, L, M = v.shape
        C = chunks if (chunks > 1 and sensors is None and all(_chunkable(t, B, L) for t in (v, lambda_v, k, q))) else 1
        ctx.chunks = C
        if C > 1:
            # time-parallel: the chunks of every sequence run as B*C batch entries from exact start states
            vc, lc, kc, qc = (_as_chunks(t, C) for t in (v, lambda_v, k, q))
            agg = slab_aggregate(vc, lc, kc, a, p)
            lam_in, eta_in = chunk_fold(agg, C, lam0, eta0, adjoint=False)
            y, y_var, lam_all, eta_all, ckpt = _launch_fwd(
                vc, lc, kc, qc, a, p, lam_in, eta_in, prior, out_dtype, need_grad)
            S = k.shape[2]
            lam_fin = lam_all.view(B, C, M, S)[:, C - 1]  # views: the last chunk's posterior is the sequence's
            eta_fin = eta_all.view(B, C, M, S)[:, C - 1]
            ctx.save_for_backward(v, lambda_v, k, q, a, p, lam0, eta0, ckpt, lam_in, eta_in)
            y, y_var = y.view(B, L, M), y_var.view(B, L, M)
        else:
            y, y_var, lam_fin, eta_fin, ckpt = _launch_fwd(
                v, lambda_v, k, q, a, p, lam0, eta0, prior, out_dtype, need_grad, sensors)
            ctx.save_for_backward(v, lambda_v, k, q, a, p, lam0, eta0, ckpt)
        ctx.prior = prior
        ctx.sensors = sensors
        ctx.out_dtype = out_dtype
        return y, y_var, lam_fin, eta_fin

    @staticmethod
    @torch.autograd.function.once_differentiable  # the hand-written gradients have no graph: a double backward raises
    def backward(ctx, dy, dy_var, dlam_fin, deta_fin):
        v, lambda_v, k, q, a, p, lam0, eta0, ckpt, *chunk_state = ctx.saved_tensors
        B, L, M = v.shape
        S = k.shape[2]
        dev = v.device
        od = ctx.out_dtype

        def grad_in(g):
            if g is None:
                return None
            if g.dtype != od:
                g = g.to(od)
            return _rowmajor_last(g)

        dy = grad_in(dy)
        dy_var = grad_in(dy_var)
        if dy is None:
            dy = torch.zeros((B, L, M), device=dev, dtype=od)
        if (dlam_fin is None) != (deta_fin is None):
            z = torch.zeros((B, M, S), device=dev, dtype=torch.float32)
            dlam_fin = z if dlam_fin is None else dlam_fin
            deta_fin = z if deta_fin is None else deta_fin
        if dlam_fin is not None:
            dlam_fin = dlam_fin.float().contiguous()
            deta_fin = deta_fin.float().contiguous()
        C = ctx.chunks
        if C > 1:
            lam_in, eta_in = chunk_state
            if not (_chunkable(dy, B, L) and _chunkable(dy_var, B, L)):
                dy = dy.contiguous()
                dy_var = None if dy_var is None else dy_var.contiguous()
            vc, lc, kc, qc, dyc, dyvc = (_as_chunks(t, C) for t in (v, lambda_v, k, q, dy, dy_var))
            adj = slab_aggregate(vc, lc, kc, a, p, q=qc, dy=dyc, dy_var=dyvc, lam0=lam_in, eta0=eta_in, prior=ctx.prior)
            dlam_seed, deta_seed = chunk_fold(adj, C, dlam_fin, deta_fin, adjoint=True)
            dv, dlv, dk, dq, da, dp, dlam_all, deta_all = _launch_bwd(
                vc, lc, kc, qc, a, p, lam_in, eta_in, ckpt, dyc, dyvc, dlam_seed, deta_seed, ctx.prior, od)
            dv, dlv = dv.view(B, L, M), dlv.view(B, L, M)
            dk, dq = dk.view(B, L, S), dq.view(B, L, S)
            dlam0 = dlam_all.view(B, C, M, S)[:, 0]
            deta0 = deta_all.view(B, C, M, S)[:, 0]
        else:
            dv, dlv, dk, dq, da, dp, dlam0, deta0 = _launch_bwd(
                v, lambda_v, k, q, a, p, lam0, eta0, ckpt, dy, dy_var, dlam_fin, deta_fin, ctx.prior, od, ctx.sensors)
        if k.dtype != torch.float32:
            dk, dq = dk.to(k.dtype), dq.to(k.dtype)
        has_state = lam0 is not None
        return (dv, dlv, dk, dq, da, dp,
                dlam0 if has_state else None, deta0 if has_state else None, None, None, None, None)


class _KLAScanEpilogueB200(torch.autograd.Function):
    """The scan with the layer's output path inside (kla_layer.py:329-338), for training: the forward kernel
    applies skip and gate at its store and also keeps the scan's own y, y_var; the backward runs the path's
    adjoint (one memory-bound kernel) and then the scan's backward kernel."""

    @staticmethod
    def forward(ctx, v, lambda_v, k, q, a, p, lam0, eta0, z, gate, skip, prior, out_dtype, sensors, gate_act):
        need_grad = any(ctx.needs_input_grad[:11])
        B, L, M = v.shape
        epi = {}
        skip_flat = None
        if skip is not None:
            skip_flat = skip.detach().float().reshape(-1).contiguous()
            epi.update(z=z, lambda_skip=skip_flat)
        if gate is not None:
            epi.update(gate=gate, gate_activation=gate_act)
        raw = None
        if need_grad and gate is not None:
            raw = (torch.empty((B, L, M), device=v.device, dtype=out_dtype), torch.empty((B, L, M), device=v.device, dtype=out_dtype))
        y, y_var, lam_fin, eta_fin, ckpt = _launch_fwd(v, lambda_v, k, q, a, p, lam0, eta0, prior, out_dtype, need_grad,
                                                       sensors, epi, raw)
        ctx.save_for_backward(v, lambda_v, k, q, a, p, lam0, eta0, ckpt, z, gate, skip_flat, *(raw or ()))
        ctx.prior, ctx.sensors, ctx.out_dtype, ctx.gate_act = prior, sensors, out_dtype, gate_act
        ctx.skip_shape, ctx.skip_dtype = (None, None) if skip is None else (skip.shape, skip.dtype)
        return y, y_var, lam_fin, eta_fin

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dout, dout_var, dlam_fin, deta_fin):
        v, lambda_v, k, q, a, p, lam0, eta0, ckpt, z, gate, skip_flat, *raw = ctx.saved_tensors
        B, L, M = v.shape
        S = k.shape[2]
        dev, od = v.device, ctx.out_dtype
        lib = _lib.load()

        def grad_in(g):
            return None if g is None else _rowmajor_last(g if g.dtype == od else g.to(od))

        dout, dout_var = grad_in(dout), grad_in(dout_var)
        if dout is None:
            dout = torch.zeros((B, L, M), device=dev, dtype=od)
        dy = torch.empty((B, L, M), device=dev, dtype=od)
        dy_var = torch.empty((B, L, M), device=dev, dtype=od)
        dz = None if z is None else torch.empty((B, L, M), device=dev, dtype=v.dtype)
        dgate = None if gate is None else torch.empty((B, L, M), device=dev, dtype=v.dtype)
        dskip = None if skip_flat is None else torch.empty_like(skip_flat)
        args = EpilogueBwdArgs(
            B=B, L=L, M=M, in_dtype=_dt(v.dtype), out_dtype=_dt(od),
            gate_activation=_lib.ACT[ctx.gate_act if gate is not None else None],
            lambda_skip_len=0 if skip_flat is None else skip_flat.numel(),
            dout=_t3(dout), dout_var=_t3(dout_var), y_raw=_t3(raw[0] if raw else None), y_var_raw=_t3(raw[1] if raw else None),
            z=_t3(z), gate=_t3(gate), lambda_skip=_ptr(skip_flat),
            dy=_t3(dy), dy_var=_t3(dy_var), dz=_t3(dz), dgate=_t3(dgate), dlambda_skip=_ptr(dskip))
        with _on(dev):
            _lib.check(lib.kla_b200_epilogue_bwd(ctypes.byref(args), _stream(dev)))
        if (dlam_fin is None) != (deta_fin is None):
            zero = torch.zeros((B, M, S), device=dev, dtype=torch.float32)
            dlam_fin = zero if dlam_fin is None else dlam_fin
            deta_fin = zero if deta_fin is None else deta_fin
        if dlam_fin is not None:
            dlam_fin, deta_fin = dlam_fin.float().contiguous(), deta_fin.float().contiguous()
        dv, dlv, dk, dq, da, dp, dlam0, deta0 = _launch_bwd(
            v, lambda_v, k, q, a, p, lam0, eta0, ckpt, dy, dy_var, dlam_fin, deta_fin, ctx.prior, od, ctx.sensors)
        if k.dtype != torch.float32:
            dk, dq = dk.to(k.dtype), dq.to(k.dtype)
        has_state = lam0 is not None
        return (dv, dlv, dk, dq, da, dp, dlam0 if has_state else None, deta0 if has_state else None,
                dz, dgate, None if dskip is None else dskip.reshape(ctx.skip_shape).to(ctx.skip_dtype), None, None, None, None)


def kla_scan_b200(
    v: torch.Tensor,
    lambda_v: torch.Tensor,
    k: torch.Tensor,
    q: torch.Tensor,
    a: torch.Tensor,
    p: torch.Tensor,
    initial_state=None,
    decode_from_prior: bool = False,
    *,
    out_dtype: Optional[torch.dtype] = None,
    log_variance: Optional[tuple] = None,
    epilogue: Optional[dict] = None,
    time_chunks: Optional[int] = None,
):
    """B200 KLA scan. Same call and return contract as the reference's
    ``kla_scan_torch`` (src/kla/ops/kla_ops.py:188-290): returns
    ``(y, y_var, KLAState)``, float32 unless ``out_dtype`` says otherwise.

    float32 inputs are read in place through their strides (the layer hands the
    scan ``torch.split`` views, src/kla/layers/kla_layer.py:205-207); bfloat16
    inputs are read as bfloat16 and widened in registers, where the reference
    widens them with a copy (kla_ops.py:126-137). ``out_dtype=torch.bfloat16``
    (bfloat16 inputs only) also writes y, y_var as bfloat16 -- what the layer
    would cast them to anyway (kla_layer.py:329-330).

    ``log_variance=(obs_var_min, obs_var_max or None)`` fuses the layer's sensor
    prologue (kla_layer.py:224-231): the ``lambda_v`` argument then holds the
    sensor projection's raw log-variance output ``x``, the kernels form
    ``1 / min(softplus(x) + obs_var_min, obs_var_max)`` in float32 on the way in,
    and the gradient returned for that argument is the one with respect to ``x``.

    ``epilogue=dict(z=, lambda_skip=, gate=, gate_activation="silu")`` fuses the
    layer's output path (kla_layer.py:329-338): ``y += lambda_skip * z``
    (``lambda_skip``: one value or one per channel), then ``y *= g``, ``y_var *= g**2``
    with ``g = act(gate)``; either half may be left out. Differentiable with respect
    to ``z``, ``gate`` and ``lambda_skip`` as well: when a gradient is needed the
    forward also keeps the scan's own y, y_var, and the backward runs the path's
    adjoint as one memory-bound kernel before the scan's backward kernel.

    ``time_chunks``: the time-parallel form of the scan. The reference's parallel
    path scans trace-normalised Moebius matrices and affine pairs over time
    (kla_ops.py:76-123, 248, 274-280); here the sequence is cut into C chunks,
    one pass composes each chunk's map on the filter state, a short fold over the
    chunks gives every chunk its exact start state, and the chunks then run
    through the ordinary kernels side by side (the backward does the same with
    the adjoint carry). ``None`` picks C from the shape (:func:`pick_time_chunks`:
    1 unless B*M is too small to fill the GPU), ``1`` switches it off.
    """
    _require_device(v)
    if a.dim() != 2:
        raise _unsupported("expects a/p of shape [M, S]")
    if v.dim() != 3 or k.dim() != 3:
        raise ValueError("v, lambda_v must be [B, L, M] and k, q [B, L, S]")
    B, L, M = v.shape
    S = k.shape[2]
    if lambda_v.shape != v.shape or q.shape != k.shape or k.shape[:2] != (B, L):
        raise ValueError("shape mismatch between v, lambda_v [B,L,M] and k, q [B,L,S]")
    if tuple(a.shape) != (M, S) or tuple(p.shape) != (M, S):
        raise ValueError(f"a and p must be [M, S] = [{M}, {S}]")
    if S > MAX_DSTATE:
        raise _unsupported(f"supports d_state <= {MAX_DSTATE} (got {S})")
    tensors = (v, lambda_v, k, q, a, p)
    if any(t.dtype == torch.float64 for t in tensors):
        raise _unsupported("runs in float32 only (float64 inputs are for gradcheck on the torch backend)")
    if any(t.device != v.device for t in tensors):
        raise ValueError("all inputs must be on the same device")

    if all(t.dtype == torch.bfloat16 for t in (v, lambda_v, k, q)):
        act = torch.bfloat16
    else:
        act = torch.float32
    if out_dtype is None:
        out_dtype = torch.float32
    if out_dtype not in (torch.float32, torch.bfloat16) or (out_dtype == torch.bfloat16 and act != torch.bfloat16):
        raise _unsupported("writes float32 outputs, or bfloat16 outputs for bfloat16 inputs")
    v, lambda_v, k, q = (_rowmajor_last(t if t.dtype == act else t.to(act)) for t in (v, lambda_v, k, q))
    a = a.float().contiguous()
    p = p.float().contiguous()
    lam0 = eta0 = None
    if initial_state is not None:
        lam0, eta0 = initial_state
        if tuple(lam0.shape) != (B, M, S) or tuple(eta0.shape) != (B, M, S):
            raise ValueError(f"initial_state must hold [B, M, S] = [{B}, {M}, {S}] tensors")
        lam0 = lam0.float().contiguous()
        eta0 = eta0.float().contiguous()

    if log_variance is not None:
        if len(log_variance) != 2 or not log_variance[0] >= 0.0:
            raise ValueError("log_variance must be (obs_var_min >= 0, obs_var_max or None)")
        log_variance = (float(log_variance[0]), None if log_variance[1] is None else float(log_variance[1]))
    if epilogue:
        epi = dict(epilogue)
        unknown = set(epi) - {"z", "lambda_skip", "gate", "gate_activation"}
        if unknown:
            raise ValueError(f"unknown epilogue keys {sorted(unknown)}")
        if (epi.get("lambda_skip") is None) != (epi.get("z") is None):
            raise ValueError("epilogue needs z and lambda_skip together")
        for name in ("z", "gate"):
            t = epi.get(name)
            if t is not None:
                if tuple(t.shape) != (B, L, M):
                    raise ValueError(f"epilogue {name} must be [B, L, M]")
                epi[name] = _rowmajor_last(t if t.dtype == act else t.to(act))
        skip = epi.get("lambda_skip")
        if skip is not None:
            if skip.numel() not in (1, M):
                raise ValueError("lambda_skip must hold one value or one per channel")
            if skip.device != v.device:
                skip = skip.to(v.device)
        gate_act = epi.get("gate_activation", "silu")
        if gate_act not in ("silu", "gelu", "relu"):
            raise ValueError("gate_activation must be 'silu', 'gelu' or 'relu'")
        y, y_var, lam_fin, eta_fin = _KLAScanEpilogueB200.apply(
            v, lambda_v, k, q, a, p, lam0, eta0, epi.get("z"), epi.get("gate"), skip, bool(decode_from_prior),
            out_dtype, log_variance, gate_act)
        return y, y_var, _state_cls()(lam=lam_fin, eta=eta_fin)
    chunks = pick_time_chunks(B, L, M, S, time_chunks) if L > 0 else 1
    y, y_var, lam_fin, eta_fin = _KLAScanB200.apply(
        v, lambda_v, k, q, a, p, lam0, eta0, bool(decode_from_prior), out_dtype, log_variance, chunks)
    return y, y_var, _state_cls()(lam=lam_fin, eta=eta_fin)


def kla_step_b200(
    v: torch.Tensor,
    lambda_v: torch.Tensor,
    k: torch.Tensor,
    q: torch.Tensor,
    a: torch.Tensor,
    p: torch.Tensor,
    state,
    decode_from_prior: bool = False,
    *,
    inplace: bool = False,
):
    """One decode step on the B200: ``kla_step`` of the reference
    (src/kla/ops/kla_ops.py:293-331). v, lambda_v: [B, M]; k, q: [B, S];
    state: (lam, eta) [B, M, S]. Returns ``(y [B,M], y_var [B,M], new_state)``.

    ``inplace=True`` updates the state tensors where they are (they must be
    float32 and contiguous) instead of allocating new ones. When a gradient is
    required the step is run as a length-1 scan, which has a backward. The two
    routes differ where the reference's own ``kla_step`` and ``kla_scan`` differ:
    the step kernel floors ``phi`` at 1e-12 and clamps the variance
    (kla_ops.py:310-312, 323), the scan leaves ``phi`` unfloored (kla_ops.py:238);
    the values agree except for keys that are zero to within 1e-6.
    """
    _require_device(v)
    if v.dim() != 2 or k.dim() != 2:
        raise ValueError("v, lambda_v must be [B, M] and k, q [B, S]")
    lam, eta = state
    if torch.is_grad_enabled() and any(
        t.requires_grad for t in (v, lambda_v, k, q, a, p, lam, eta)
    ):
        y, y_var, st = kla_scan_b200(
            v.unsqueeze(1), lambda_v.unsqueeze(1), k.unsqueeze(1), q.unsqueeze(1), a, p,
            initial_state=(lam, eta), decode_from_prior=decode_from_prior)
        return y[:, 0], y_var[:, 0], st
    B, M = v.shape
    S = k.shape[1]
    if tuple(a.shape) != (M, S) or tuple(p.shape) != (M, S) or tuple(lam.shape) != (B, M, S):
        raise ValueError("shape mismatch between v [B,M], k [B,S], a/p [M,S] and the state [B,M,S]")
    if S > MAX_DSTATE:
        raise _unsupported(f"supports d_state <= {MAX_DSTATE} (got {S})")
    if any(t.dtype == torch.float64 for t in (v, lambda_v, k, q, a, p, lam, eta)):
        raise _unsupported("runs in float32 only")
    lib = _lib.load()
    act = torch.bfloat16 if all(t.dtype == torch.bfloat16 for t in (v, lambda_v, k, q)) else torch.float32

    def row(t):
        t = t if t.dtype == act else t.to(act)
        return t if (t.shape[-1] <= 1 or t.stride(-1) == 1) else t.contiguous()

    v, lambda_v, k, q = row(v), row(lambda_v), row(k), row(q)
    a = a.float().contiguous()
    p = p.float().contiguous()
    if inplace:
        if lam.dtype != torch.float32 or not lam.is_contiguous() or eta.dtype != torch.float32 or not eta.is_contiguous():
            raise ValueError("inplace=True needs float32 contiguous state tensors")
        lam_out, eta_out = lam, eta
    else:
        lam, eta = lam.float().contiguous(), eta.float().contiguous()
        lam_out, eta_out = torch.empty_like(lam), torch.empty_like(eta)
    dev = v.device
    y = torch.empty((B, M), device=dev, dtype=torch.float32)
    y_var = torch.empty((B, M), device=dev, dtype=torch.float32)
    args = StepArgs(
        B=B, M=M, S=S, in_dtype=_dt(act), out_dtype=F32, decode_from_prior=int(decode_from_prior),
        v=_ptr(v), lambda_v=_ptr(lambda_v), v_stride_b=v.stride(0), lambda_v_stride_b=lambda_v.stride(0),
        k=_ptr(k), q=_ptr(q), k_stride_b=k.stride(0), q_stride_b=q.stride(0),
        a=_ptr(a), p=_ptr(p), lam=_ptr(lam), eta=_ptr(eta),
        y=_ptr(y), y_var=_ptr(y_var), lam_out=_ptr(lam_out), eta_out=_ptr(eta_out),
    )
    with _on(dev):
        _lib.check(lib.kla_b200_step(ctypes.byref(args), _stream(dev)))
    return y, y_var, _state_cls()(lam=lam_out, eta=eta_out)
