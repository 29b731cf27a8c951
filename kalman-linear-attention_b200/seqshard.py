"""Sequence-sharded scan: the time axis split into slabs, one per GPU.

For sequences long enough that one GPU's time loop is the bottleneck, rank r
holds the r-th slab ``[B, L_r, ...]`` of v, lambda_v, k, q (and gets the r-th
slab of y, y_var). The reference has no such mode (its only tool for long
sequences is carrying state between calls, tests/test_ops.py:63-75); what
makes one possible is that a slab acts on the filter state through an
associative map (src/kla/ops/kla_ops.py:76-116).

Forward, per rank: (1) the slab's state map as a 7-number aggregate
(``kla_b200_slab_aggregate``, one pass over v, lambda_v, k); (2) one
all-gather of the aggregates (28 B per lane and rank); (3) fold the maps of the
earlier ranks onto the initial state -- a few elementwise float64 operations on
[B, M, S]; (4) the ordinary fused scan from that exact state. The posterior of
the last rank is broadcast as the returned state.

Backward, per rank: (1) the slab's adjoint aggregate (one forward-time pass
with dy, dy_var and the true initial state): the carry leaving the slab is an
upper-triangular affine function of the carry entering it; (2) one all-gather;
(3) fold the later ranks' maps onto the gradient of the returned state;
(4) the ordinary fused backward seeded with that carry; (5) all-reduce of da,
dp, which sum over time. dk, dq, dv, dlambda_v are local to the slab.

The collectives are NCCL through ``torch.distributed`` (gloo in the CPU
tests); gathered tensors land in this GPU's memory and are read from there.
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from . import ops


# ------------------------------------------------------------------ kernels

slab_aggregate = ops.slab_aggregate  # the launch lives with the other kernel launches


# -------------------------------------------------------- folds (pure torch)

def prefix_state(aggs: Sequence[torch.Tensor], lam0: Optional[torch.Tensor], eta0: Optional[torch.Tensor],
                 shape: Tuple[int, int, int], device) -> Tuple[torch.Tensor, torch.Tensor]:
    """State a slab starts from: the earlier slabs' maps (in time order) applied
    to the initial state. Returns float32 (lam, eta)."""
    f64 = dict(device=device, dtype=torch.float64)
    if lam0 is None:
        P, mean = torch.ones(shape, **f64), torch.zeros(shape, **f64)
    else:
        P = 1.0 / lam0.to(**f64).clamp_min(1e-20)
        mean = eta0.to(**f64) * P
    for A in aggs:
        A = A.to(torch.float64)
        x = A[..., 0] + A[..., 1] * P
        w = A[..., 2] + A[..., 3] * P
        z = A[..., 4] + A[..., 5] * P + A[..., 6] * mean
        P, mean = w / x, z / x
    lam = 1.0 / P
    return lam.float(), (mean * lam).float()


def carry_from_state_grad(dlam, deta, P_end, mean_end):
    """(dL/dP, dL/dmean) at the end of the sequence from the gradient of the
    returned (lam, eta) = (1/P, mean/P)."""
    lam = 1.0 / P_end
    eta = mean_end * lam
    return -lam * (lam * dlam + eta * deta), deta * lam


def state_grad_from_carry(cP, cm, P_end, mean_end):
    """Inverse of :func:`carry_from_state_grad`: the (dlam, deta) seed that makes
    the backward kernel start from the carry (cP, cm)."""
    deta = cm * P_end
    dlam = -(cP * P_end * P_end + mean_end * deta)
    return dlam, deta


def suffix_carry(adjs: Sequence[torch.Tensor], cP: torch.Tensor, cm: torch.Tensor):
    """Carry entering a slab at its end: the later slabs' adjoint maps applied,
    last slab first, to the carry at the end of the sequence. ``adjs`` is in
    time order (the slab right after this one first)."""
    for A in reversed(list(adjs)):
        A = A.to(torch.float64)
        cP, cm = A[..., 0] * cP + A[..., 1] * cm + A[..., 3], A[..., 2] * cm + A[..., 4]
    return cP, cm


# ------------------------------------------------------------- collectives

def _world(group):
    if not (dist.is_available() and dist.is_initialized()):
        return 0, 1
    return dist.get_rank(group), dist.get_world_size(group)


def _all_gather(x: torch.Tensor, group) -> List[torch.Tensor]:
    rank, world = _world(group)
    if world == 1:
        return [x]
    out = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(out, x.contiguous(), group=group)
    return out


def _global_rank(group, group_rank: int) -> int:
    return dist.get_global_rank(group, group_rank) if group is not None else group_rank


class _SeqShardedScan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, v, lambda_v, k, q, a, p, lam0, eta0, prior: bool, out_dtype, group):
        rank, world = _world(group)
        B, L, M = v.shape
        S = k.shape[2]
        agg = slab_aggregate(v, lambda_v, k, a, p)
        gathered = _all_gather(agg, group)
        lam_in, eta_in = prefix_state(gathered[:rank], lam0, eta0, (B, M, S), v.device)
        need_grad = any(ctx.needs_input_grad[:8])
        y, y_var, lam_fin, eta_fin, ckpt = ops._launch_fwd(
            v, lambda_v, k, q, a, p, lam_in.contiguous(), eta_in.contiguous(), prior, out_dtype, need_grad)
        # the sequence's posterior is the last slab's; every rank returns it
        lam_out, eta_out = lam_fin.clone(), eta_fin.clone()
        if world > 1:
            src = _global_rank(group, world - 1)
            dist.broadcast(lam_out, src=src, group=group)
            dist.broadcast(eta_out, src=src, group=group)
        ctx.save_for_backward(v, lambda_v, k, q, a, p, lam_in, eta_in, ckpt, lam_out, eta_out)
        ctx.prior, ctx.out_dtype, ctx.group = prior, out_dtype, group
        ctx.has_state = lam0 is not None
        return y, y_var, lam_out, eta_out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dy, dy_var, dlam_fin, deta_fin):
        v, lambda_v, k, q, a, p, lam_in, eta_in, ckpt, lam_out, eta_out = ctx.saved_tensors
        group, od = ctx.group, ctx.out_dtype
        rank, world = _world(group)
        B, L, M = v.shape
        S = k.shape[2]
        dev = v.device

        def grad_in(g):
            if g is None:
                return None
            return ops._rowmajor_last(g if g.dtype == od else g.to(od))

        dy, dy_var = grad_in(dy), grad_in(dy_var)
        if dy is None:
            dy = torch.zeros((B, L, M), device=dev, dtype=od)
        adj = slab_aggregate(v, lambda_v, k, a, p, q=q, dy=dy, dy_var=dy_var,
                             lam0=lam_in.contiguous(), eta0=eta_in.contiguous(), prior=ctx.prior)
        gathered = _all_gather(adj, group)
        # gradient of the returned state: every rank holds a copy of that output, so
        # the copies' gradients add
        f64 = dict(device=dev, dtype=torch.float64)
        dl = torch.zeros((B, M, S), **f64) if dlam_fin is None else dlam_fin.to(**f64)
        de = torch.zeros((B, M, S), **f64) if deta_fin is None else deta_fin.to(**f64)
        if world > 1:
            dist.all_reduce(dl, group=group)
            dist.all_reduce(de, group=group)
        P_last = 1.0 / lam_out.to(**f64)
        cP, cm = carry_from_state_grad(dl, de, P_last, eta_out.to(**f64) * P_last)
        cP, cm = suffix_carry(gathered[rank + 1:], cP, cm)
        mine = gathered[rank].to(torch.float64)
        dlam_seed, deta_seed = state_grad_from_carry(cP, cm, mine[..., 5], mine[..., 6])
        dv, dlv, dk, dq, da, dp, dlam0, deta0 = ops._launch_bwd(
            v, lambda_v, k, q, a, p, lam_in.contiguous(), eta_in.contiguous(), ckpt, dy, dy_var,
            dlam_seed.float().contiguous(), deta_seed.float().contiguous(), ctx.prior, od)
        if world > 1:
            dist.all_reduce(da, group=group)  # sums over time cross the slabs
            dist.all_reduce(dp, group=group)
            src = _global_rank(group, 0)      # the initial state belongs to the first slab
            dist.broadcast(dlam0, src=src, group=group)
            dist.broadcast(deta0, src=src, group=group)
        if k.dtype != torch.float32:
            dk, dq = dk.to(k.dtype), dq.to(k.dtype)
        hs = ctx.has_state
        return dv, dlv, dk, dq, da, dp, (dlam0 if hs else None), (deta0 if hs else None), None, None, None


def kla_scan_seq_sharded(v, lambda_v, k, q, a, p, initial_state=None, decode_from_prior: bool = False, *,
                         group=None, out_dtype: Optional[torch.dtype] = None):
    """Scan this rank's time slab of a sequence split over the ranks of ``group``
    (rank order = time order). Same contract as ``kla_scan_b200`` per slab; the
    returned state is the posterior after the LAST slab, on every rank.
    ``initial_state`` is the state before the FIRST slab and must be the same on
    every rank (or None for the unit prior). Without an initialised process
    group this is the single-GPU scan computed through the same code."""
    ops._require_device(v)
    B, L, M = v.shape
    S = k.shape[2]
    act = torch.bfloat16 if all(t.dtype == torch.bfloat16 for t in (v, lambda_v, k, q)) else torch.float32
    out_dtype = out_dtype or torch.float32
    v, lambda_v, k, q = (ops._rowmajor_last(t if t.dtype == act else t.to(act)) for t in (v, lambda_v, k, q))
    a, p = a.float().contiguous(), p.float().contiguous()
    lam0 = eta0 = None
    if initial_state is not None:
        lam0, eta0 = (t.float().contiguous() for t in initial_state)
    y, y_var, lam, eta = _SeqShardedScan.apply(v, lambda_v, k, q, a, p, lam0, eta0,
                                               bool(decode_from_prior), out_dtype, group)
    return y, y_var, ops._state_cls()(lam=lam, eta=eta)
