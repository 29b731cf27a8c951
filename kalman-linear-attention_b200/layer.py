"""The reference layer's forward with the scan's neighbours inside the scan kernels.

``KLALayer.forward`` (src/kla/layers/kla_layer.py:295-349) surrounds the scan with
elementwise passes over ``[B, L, M]`` tensors: widening casts of ``v`` and of the
log-variances, ``softplus``, floor, ceiling and reciprocal (``_project_sensors``,
kla_layer.py:224-231), and after the scan two narrowing casts, the skip path and
the gate (kla_layer.py:329-338) -- and autograd's backward of each of them.
``fused_forward`` is the same function of the same parameters with those passes
folded into ``kla_scan_b200``: the kernels read the sensor projection's slices in
the activation dtype, form the precision in registers, and apply skip and gate
where they store ``y``; the backward is the epilogue's adjoint kernel followed by
the scan's backward kernel. The causal convolution in front of the sensor
projection (``CausalConv1d``, src/kla/layers/common.py:57-96: transpose, cat,
``conv1d``, activation, transpose back, and autograd's backward of each) runs as one
kernel per direction in the layer's own ``[B, L, D]`` layout (``causal_conv_b200``).
The projections stay the layer's own modules.

``enable()`` rebinds ``KLALayer.forward`` so that layers configured with
``backend="b200"`` take this route for sequences on an sm_100 GPU; every other
call (another backend, CPU tensors, float64, the single-token decode route) goes
to the original method. ``disable()`` restores it.
"""

from __future__ import annotations

import ctypes
import sys

import torch
import torch.nn.functional as F

from . import _lib
from .ops import _on, _rowmajor_last, _stream, _t3, kla_scan_b200

_ORIG_FORWARD = None


class _CausalConvB200(torch.autograd.Function):
    """``CausalConv1d.forward`` (common.py:87-96) on ``[B, L, D]`` tensors: ``kla_b200_conv_seq`` forward,
    ``kla_b200_conv_seq_bwd`` backward (the pre-activation is recomputed from ``x``)."""

    @staticmethod
    def forward(ctx, x, weight, bias, state, activation):
        B, L, D = x.shape
        K = weight.shape[-1]
        lib = _lib.load()
        w = weight.detach().float().reshape(D, K).contiguous()
        b = None if bias is None else bias.detach().float().contiguous()
        x = _rowmajor_last(x)
        if state is None:
            state = torch.zeros((B, D, K - 1), device=x.device, dtype=x.dtype)
        else:
            state = state.detach().to(x.dtype).contiguous()
        z = torch.empty((B, L, D), device=x.device, dtype=x.dtype)
        new_state = torch.empty_like(state)
        args = _lib.ConvSeqArgs(B=B, L=L, D=D, K=K, dtype=_lib.F32 if x.dtype == torch.float32 else _lib.BF16,
                                activation=_lib.ACT[activation], x=_t3(x), weight=w.data_ptr(),
                                bias=None if b is None else b.data_ptr(), state=state.data_ptr(),
                                state_out=new_state.data_ptr(), z=_t3(z))
        with _on(x.device):
            _lib.check(lib.kla_b200_conv_seq(ctypes.byref(args), _stream(x.device)))
        ctx.save_for_backward(x, w, b, state)
        ctx.activation, ctx.wshape = activation, weight.shape
        ctx.wdtype, ctx.bdtype = weight.dtype, None if bias is None else bias.dtype
        ctx.mark_non_differentiable(new_state)
        return z, new_state

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dz, _dstate):
        x, w, b, state = ctx.saved_tensors
        B, L, D = x.shape
        K = w.shape[1]
        dz = _rowmajor_last(dz if dz.dtype == x.dtype else dz.to(x.dtype))
        dx = torch.empty((B, L, D), device=x.device, dtype=x.dtype)
        dw = torch.zeros((D, K), device=x.device, dtype=torch.float32)
        db = None if b is None else torch.zeros((D,), device=x.device, dtype=torch.float32)
        args = _lib.ConvSeqBwdArgs(B=B, L=L, D=D, K=K, dtype=_lib.F32 if x.dtype == torch.float32 else _lib.BF16,
                                   activation=_lib.ACT[ctx.activation], x=_t3(x), dz=_t3(dz), weight=w.data_ptr(),
                                   bias=None if b is None else b.data_ptr(), state=state.data_ptr(), dx=_t3(dx),
                                   dweight=dw.data_ptr(), dbias=None if db is None else db.data_ptr())
        with _on(x.device):
            _lib.check(_lib.load().kla_b200_conv_seq_bwd(ctypes.byref(args), _stream(x.device)))
        return dx, dw.reshape(ctx.wshape).to(ctx.wdtype), None if db is None else db.to(ctx.bdtype), None, None


def causal_conv_b200(x: torch.Tensor, weight: torch.Tensor, bias, state=None, activation: str = "silu"):
    """Depthwise causal convolution over time with its activation, ``x`` ``[B, L, D]`` float32 or bfloat16,
    ``weight`` ``[D, 1, K]`` (``K <= 8``), ``state`` the ``K-1`` inputs before the sequence (``[B, D, K-1]``, zeros
    when None). Returns ``(z [B, L, D], new_state)`` like the reference module; differentiable with respect to
    ``x``, ``weight`` and ``bias`` (the carried window is treated as a constant)."""
    return _CausalConvB200.apply(x, weight, bias, state, activation)


def _conv(layer, z, conv_state):
    """The layer's convolution: the B200 kernels where they apply, the layer's own module otherwise."""
    conv, cfg = layer.conv, layer.config
    if (z.dtype in (torch.float32, torch.bfloat16) and conv.kernel_size <= _lib.MAX_CONV_TAPS
            and cfg.conv_activation in ("silu", "gelu", "relu")
            and not (conv_state is not None and conv_state.requires_grad and torch.is_grad_enabled())):
        return causal_conv_b200(z, conv.weight, conv.bias, conv_state, cfg.conv_activation)
    return conv(z, conv_state)


def _fusable(layer, x: torch.Tensor, state) -> bool:
    cfg = layer.config
    if getattr(cfg, "backend", None) != "b200" or not x.is_cuda or x.dtype == torch.float64:
        return False
    if torch.cuda.get_device_capability(x.device)[0] != 10:
        return False
    if state is not None and x.shape[1] == 1:  # decode by one token: kla_step, not the scan
        return False
    return cfg.gating_activation in ("silu", "gelu", "relu") or not cfg.use_gating


def fused_forward(layer, x: torch.Tensor, state=None, return_state: bool = False):
    """``layer(x, state, return_state)`` for a reference ``KLALayer`` and ``L > 1`` (or no state), computed
    with the sensor prologue and the skip/gate epilogue inside the B200 scan kernels. Same returns as
    the reference method: ``out`` or ``(out, out_var)``, with the new ``KLALayerState`` when asked for."""
    mod = sys.modules[type(layer).__module__]
    cfg = layer.config
    S = layer.d_state
    emit_state = return_state or state is not None

    projected = layer.in_proj(x)
    if cfg.use_gating:
        z, gate = projected.chunk(2, dim=-1)
    else:
        z, gate = projected, None
    conv_state = state.conv if state is not None else None
    if layer.conv is not None:
        z, conv_state = _conv(layer, z, conv_state)

    # the four sensor signals, left in the dtype and memory the projection wrote them in (kla_layer.py:199-222)
    v, log_sigma_v, k, q = torch.split(layer.sensor_proj(z), [layer._w_value, layer._w_var, S, S], dim=-1)
    if layer._value_rank == "conv":
        v = z
    elif layer.value_expand is not None:
        v = layer.value_expand(v)
    if layer.var_expand is not None:
        log_sigma_v = layer.var_expand(log_sigma_v)
    if cfg.qk_norm:
        k, q = mod.l2_norm(k), mod.l2_norm(q)
    if cfg.clip_value is not None:
        k, q = k.clamp(-cfg.clip_value, cfg.clip_value), q.clamp(-cfg.clip_value, cfg.clip_value)
    # the activation dtype is the projections' (bfloat16 under autocast even when x itself is float32)
    act = torch.bfloat16 if log_sigma_v.dtype == torch.bfloat16 and v.dtype == torch.bfloat16 else torch.float32
    v, log_sigma_v, k, q = (t if t.dtype == act else t.to(act) for t in (v, log_sigma_v, k, q))

    a_bar, p_bar = layer._compute_aq()
    epilogue = {}
    if layer.lambda_skip is not None:
        epilogue.update(z=z, lambda_skip=layer.lambda_skip)
    if gate is not None:
        epilogue.update(gate=gate, gate_activation=cfg.gating_activation)
    ssm_state = state.ssm if state is not None else None

    def scan(v, log_sigma_v, k, q, a_bar, p_bar, lam0, eta0, *epi_tensors):
        epi = dict(epilogue)
        for name, t in zip([n for n in ("z", "lambda_skip", "gate") if n in epi], epi_tensors):
            epi[name] = t
        y, y_var, st = kla_scan_b200(
            v, log_sigma_v, k, q, a_bar, p_bar, initial_state=None if lam0 is None else (lam0, eta0),
            decode_from_prior=cfg.decode_from_prior, out_dtype=act,
            log_variance=(cfg.obs_var_min, cfg.obs_var_max), epilogue=epi or None)
        return y, y_var, st.lam, st.eta

    lam0 = ssm_state.lam if ssm_state is not None else None
    eta0 = ssm_state.eta if ssm_state is not None else None
    epi_tensors = [epilogue[n] for n in ("z", "lambda_skip", "gate") if n in epilogue]
    with torch.autocast(device_type=x.device.type, enabled=False):
        if cfg.checkpoint_ssm and torch.is_grad_enabled() and layer.training:
            y, y_var, lam, eta = torch.utils.checkpoint.checkpoint(
                scan, v, log_sigma_v, k, q, a_bar, p_bar, lam0, eta0, *epi_tensors, use_reentrant=False)
        else:
            y, y_var, lam, eta = scan(v, log_sigma_v, k, q, a_bar, p_bar, lam0, eta0, *epi_tensors)
    if not torch.is_autocast_enabled(x.device.type):
        # kla_layer.py:329-330; under autocast the projection below rounds its input to the autocast dtype itself
        y, y_var = y.to(x.dtype), y_var.to(x.dtype)

    out = layer.out_proj(y)
    result = (out, F.linear(y_var, layer.out_proj.weight.pow(2))) if cfg.return_variance else out
    if emit_state:
        return result, mod.KLALayerState(conv=conv_state, ssm=mod.KLAState(lam=lam, eta=eta))
    return result


def enable() -> None:
    """Route ``KLALayer.forward`` of the importable reference package through :func:`fused_forward` where it
    applies (see the module docstring); idempotent."""
    import kla.layers.kla_layer as kla_layer

    global _ORIG_FORWARD
    if _ORIG_FORWARD is not None:
        return
    _ORIG_FORWARD = kla_layer.KLALayer.forward
    orig = _ORIG_FORWARD

    def forward(self, x, state=None, return_state=False):
        if _fusable(self, x, state):
            return fused_forward(self, x, state, return_state)
        return orig(self, x, state, return_state)

    forward.__doc__ = orig.__doc__
    kla_layer.KLALayer.forward = forward


def disable() -> None:
    import kla.layers.kla_layer as kla_layer

    global _ORIG_FORWARD
    if _ORIG_FORWARD is not None:
        kla_layer.KLALayer.forward = _ORIG_FORWARD
        _ORIG_FORWARD = None
