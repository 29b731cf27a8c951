"""Forward + backward of the scan for batches that live in HOST memory.

A training step whose activations arrive in pinned host buffers and whose results go back
to host buffers is bound by the PCIe link, not by the kernels: at the headline shape the
step moves 0.54 GB each way for 2.2 ms of GPU work. The scan is independent over the batch
(``y[b]`` depends on ``v[b], lambda_v[b], k[b], q[b]`` only; ``da, dp`` are sums over ``b``),
so ``scan_fwd_bwd_host`` cuts the batch into chunks and pipelines them over one copy-in
stream, a few kernel streams and one copy-out stream, tied together with events: a chunk's
forward starts when its ``v, lambda_v, k, q`` have landed (the upstream gradients follow
behind), its ``y, y_var`` leave while its backward runs, and the two copy engines work at
the same time (PCIe is full duplex) instead of copy-in, compute and copy-out taking turns.

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
    n_chunks = (B + chunk - 1) // chunk
    pool = _side_streams(device, 2 + max(1, min(n_streams, n_chunks)))
    s_in, s_out, s_cmp = pool[0], pool[1], pool[2:]  # one stream per copy engine, several for the kernels
    for s in pool:
        s.wait_stream(main)
    with torch.cuda.device(device):
        with torch.cuda.stream(s_in):
            a = host["a"].to(device, non_blocking=True)
            p = host["p"].to(device, non_blocking=True)
        partial = []  # per chunk (da, dp), added in chunk order at the end
        keep = [a, p]
        for ci, b0 in enumerate(range(0, B, chunk)):
            sc = s_cmp[ci % len(s_cmp)]
            sl = slice(b0, min(B, b0 + chunk))
            # copy-in: what the forward needs first, the upstream gradients behind it
            with torch.cuda.stream(s_in):
                g = {n: host[n][sl].to(device, non_blocking=True) for n in _IN}
                in_fwd = torch.cuda.Event()
                in_fwd.record(s_in)
                g.update({n: host[n][sl].to(device, non_blocking=True) for n in ("dy", "dyvar")})
                in_bwd = torch.cuda.Event()
                in_bwd.record(s_in)
            ins = [g[n] for n in _IN]
            with torch.cuda.stream(sc):
                sc.wait_event(in_fwd)
                y, y_var, _, _, ckpt = _launch_fwd(*ins, a, p, None, None, decode_from_prior, torch.float32, True)
                fwd_done = torch.cuda.Event()
                fwd_done.record(sc)
                sc.wait_event(in_bwd)
                dv, dlv, dk, dq, da, dp, _, _ = _launch_bwd(*ins, a, p, None, None, ckpt, g["dy"], g["dyvar"], None, None,
                                                            decode_from_prior, torch.float32)
                bwd_done = torch.cuda.Event()
                bwd_done.record(sc)
            # copy-out: y, y_var can leave while the backward runs
            with torch.cuda.stream(s_out):
                s_out.wait_event(fwd_done)
                out["y"][sl].copy_(y, non_blocking=True)
                out["y_var"][sl].copy_(y_var, non_blocking=True)
                s_out.wait_event(bwd_done)
                for name, t in (("dv", dv), ("dlambda_v", dlv), ("dk", dk), ("dq", dq)):
                    out[name][sl].copy_(t, non_blocking=True)
            partial.append((da, dp))
            # every buffer of the chunk is touched by up to three streams; tell the allocator
            for t in (*g.values(), y, y_var, ckpt, dv, dlv, dk, dq, da, dp):
                for s in (s_in, sc, s_out):
                    t.record_stream(s)
        for s in pool:
            main.wait_stream(s)
        da = torch.stack([x[0] for x in partial]).sum(0) if len(partial) > 1 else partial[0][0]
        dp = torch.stack([x[1] for x in partial]).sum(0) if len(partial) > 1 else partial[0][1]
        out["da"].copy_(da, non_blocking=True)
        out["dp"].copy_(dp, non_blocking=True)
        for t in (*keep, *(x for pr in partial for x in pr)):
            t.record_stream(main)
    return out
