"""Forward + backward of the scan for batches that live in HOST memory.

A training step whose activations arrive in pinned host buffers and whose results go back
to host buffers is bound by the PCIe link, not by the kernels: at the headline shape the
step moves 0.54 GB each way for 2.2 ms of GPU work. The scan is independent over the batch
(``y[b]`` depends on ``v[b], lambda_v[b], k[b], q[b]`` only; ``da, dp`` are sums over ``b``),
so ``scan_fwd_bwd_host`` cuts the batch into chunks and runs each chunk's
copy-in -> forward -> backward -> copy-out on its own CUDA stream. The two copy engines then
work at the same time (PCIe is full duplex) and the kernels of one chunk run under the
copies of the next, instead of copy-in, compute and copy-out taking turns.

Same kernels and same numerics as ``kla_scan_b200`` + autograd on the whole batch (float32
activations; the entry point calls the forward and backward launches directly): the chunks
are disjoint sets of lanes; only ``da, dp`` are added across chunks (in chunk order, so the
result does not depend on timing).
"""

from __future__ import annotations

import torch

from .ops import _launch_bwd, _launch_fwd, _require_sm100

_IN = ("v", "lambda_v", "k", "q")
_STREAMS: dict = {}  # device index -> side streams, created once so that the allocator's per-stream pools are reused


def _side_streams(device: torch.device, n: int):
    pool = _STREAMS.setdefault(device.index if device.index is not None else torch.cuda.current_device(), [])
    while len(pool) < n:
        pool.append(torch.cuda.Stream(device))
    return pool[:n]
_OUT = ("y", "y_var", "dv", "dlambda_v", "dk", "dq", "da", "dp")


def scan_fwd_bwd_host(host: dict, device, out: dict | None = None, chunk: int = 1, n_streams: int = 4,
                      decode_from_prior: bool = False) -> dict:
    """``host``: pinned CPU tensors ``v, lambda_v [B, L, M]``, ``k, q [B, L, S]``, ``a, p [M, S]`` and the
    upstream gradients ``dy, dyvar [B, L, M]``. Returns pinned CPU tensors ``y, y_var, dv, dlambda_v,
    dk, dq, da, dp`` (``out`` is reused when given). The call returns after queueing; the results are
    complete once the current stream of ``device`` has been synchronised."""
    device = torch.device(device)
    for name in (*_IN, "a", "p", "dy", "dyvar"):
        t = host[name]
        if t.is_cuda or not t.is_pinned():
            raise ValueError(f"scan_fwd_bwd_host takes pinned host tensors; {name} is "
                             f"{'on ' + str(t.device) if t.is_cuda else 'pageable'}")
        if t.dtype != torch.float32:
            raise NotImplementedError(f"scan_fwd_bwd_host takes float32 host tensors; {name} is {t.dtype}. "
                                      "Move the data yourself and call kla_scan_b200 for other dtypes.")
    B = host["v"].shape[0]
    if out is None:
        like = dict(y="v", y_var="v", dv="v", dlambda_v="lambda_v", dk="k", dq="q", da="a", dp="p")
        out = {n: torch.empty(host[src].shape, dtype=torch.float32 if n in ("y", "y_var", "dk", "dq", "da", "dp")
                              else host[src].dtype, pin_memory=True) for n, src in like.items()}
    _require_sm100(device)
    main = torch.cuda.current_stream(device)
    streams = _side_streams(device, max(1, min(n_streams, (B + chunk - 1) // chunk)))
    with torch.cuda.device(device):
        a = host["a"].to(device, non_blocking=True)
        p = host["p"].to(device, non_blocking=True)
        ready = torch.cuda.Event()
        ready.record(main)
        partial = []  # per chunk (da, dp), added in chunk order at the end
        for ci, b0 in enumerate(range(0, B, chunk)):
            s = streams[ci % len(streams)]
            s.wait_event(ready)
            sl = slice(b0, min(B, b0 + chunk))
            with torch.cuda.stream(s):
                g = {n: host[n][sl].to(device, non_blocking=True) for n in (*_IN, "dy", "dyvar")}
                ins = [g[n] for n in _IN]
                y, y_var, _, _, ckpt = _launch_fwd(*ins, a, p, None, None, decode_from_prior, torch.float32, True)
                dv, dlv, dk, dq, da, dp, _, _ = _launch_bwd(*ins, a, p, None, None, ckpt, g["dy"], g["dyvar"], None, None,
                                                            decode_from_prior, torch.float32)
                for name, t in (("y", y), ("y_var", y_var), ("dv", dv), ("dlambda_v", dlv), ("dk", dk), ("dq", dq)):
                    out[name][sl].copy_(t, non_blocking=True)
                partial.append((da, dp))
        for s in streams:
            main.wait_stream(s)
        da = torch.stack([x[0] for x in partial]).sum(0) if len(partial) > 1 else partial[0][0]
        dp = torch.stack([x[1] for x in partial]).sum(0) if len(partial) > 1 else partial[0][1]
        out["da"].copy_(da, non_blocking=True)
        out["dp"].copy_(dp, non_blocking=True)
        for t in (a, p):
            for s in streams:
                t.record_stream(s)
    return out
