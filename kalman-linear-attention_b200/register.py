"""Plug the ``b200`` backend into an importable reference package ``kla``
without editing it.

``kla_scan`` looks its backend up by name in the module-level dict
``kla.ops.kla_ops._BACKENDS`` (src/kla/ops/kla_ops.py:430-442, 509-516), and
``KLAConfig.backend`` is passed straight through by the layer
(src/kla/layers/kla_layer.py:241-257), so one dict entry makes
``kla_scan(..., backend="b200")``, ``KLALayer(.., KLAConfig(backend="b200"))``
and ``SequenceModel`` all run the B200 kernels. ``"auto"`` keeps resolving as
before (kla_ops.py:466-483).

Single-token decode has no dispatch: the layer calls the name ``kla_step`` it
imported (kla_layer.py:39, 277-293). ``register(decode_hook=True)`` rebinds
that name to a function that runs the B200 step kernel for CUDA tensors on an
sm_100 device and calls the original for everything else.
"""

from __future__ import annotations

import torch

from . import layer as fused_layer
from . import ops

_ORIG_STEP = None


def register(name: str = "b200", decode_hook: bool = True, fuse_layer: bool = False) -> None:
    """``fuse_layer=True`` also routes ``KLALayer.forward`` through ``layer.fused_forward`` for layers whose
    config says ``backend="b200"`` (sensor prologue and skip/gate epilogue inside the scan kernels)."""
    import kla  # the reference package; ImportError if it is not installed
    import kla.layers.kla_layer as kla_layer
    import kla.ops as kla_ops_pkg
    import kla.ops.kla_ops as kla_ops

    kla_ops._BACKENDS[name] = ops.kla_scan_b200
    if fuse_layer:
        fused_layer.enable()

    global _ORIG_STEP
    if decode_hook and _ORIG_STEP is None:
        _ORIG_STEP = kla_ops.kla_step
        orig = _ORIG_STEP

        def kla_step(v, lambda_v, k, q, a, p, state, decode_from_prior=False):
            if (v.is_cuda and v.dtype != torch.float64
                    and torch.cuda.get_device_capability(v.device)[0] == 10):
                return ops.kla_step_b200(v, lambda_v, k, q, a, p, state,
                                         decode_from_prior=decode_from_prior)
            return orig(v, lambda_v, k, q, a, p, state, decode_from_prior=decode_from_prior)

        kla_step.__doc__ = orig.__doc__
        # kla.ops.kla_ops.kla_step itself stays: kla_scan_reference loops over it
        # (kla_ops.py:334-362) and must remain the reference.
        for mod in (kla_layer, kla_ops_pkg, kla):
            if hasattr(mod, "kla_step"):
                setattr(mod, "kla_step", kla_step)


def unregister(name: str = "b200") -> None:
    import kla
    import kla.layers.kla_layer as kla_layer
    import kla.ops as kla_ops_pkg
    import kla.ops.kla_ops as kla_ops

    kla_ops._BACKENDS.pop(name, None)
    fused_layer.disable()
    global _ORIG_STEP
    if _ORIG_STEP is not None:
        for mod in (kla_layer, kla_ops_pkg, kla):
            if hasattr(mod, "kla_step"):
                setattr(mod, "kla_step", _ORIG_STEP)
        _ORIG_STEP = None
