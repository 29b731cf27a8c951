"""Batch x channel sharding of the scan across the GPUs of one box.

The filter's lanes are independent over (batch, channel) -- ``y[b, :, m]``
depends on ``v[b, :, m]``, ``lambda_v[b, :, m]``, ``k[b]``, ``q[b]``, ``a[m]``,
``p[m]`` only -- so the forward needs no communication: each rank scans its own
block of batch elements and channels. The backward has two small sums that cross
ranks:

* ``da, dp [M, S]`` are sums over the batch: ranks that hold the same channels
  but different batch elements add theirs (all-reduce over the *batch group*);
* ``dk, dq [B, L, S]`` are sums over channels: ranks that hold the same batch
  elements but different channels add theirs (all-reduce over the *channel
  group*).

The reference has no multi-device path at all (no ``torch.distributed`` call
site anywhere in it); this module is the data-parallel layer around its scan.
Everything here is plain ``torch.distributed`` (NCCL on GPUs, gloo in the CPU
tests) and works with any scan callable of the reference's backend contract.
"""

from __future__ import annotations

import math
from typing import Callable, NamedTuple, Optional, Tuple

import torch
import torch.distributed as dist


class Block(NamedTuple):
    """The block of the [B, M] lane grid one rank owns."""

    b0: int
    b1: int
    m0: int
    m1: int
    batch_rank: int    # index along the batch split
    channel_rank: int  # index along the channel split
    batch_parts: int
    channel_parts: int


def grid_for(B: int, M: int, world: int, align: int = 32) -> Tuple[int, int]:
    """Split ``world`` ranks into (batch_parts, channel_parts). Batch is split
    first (it needs no replication of k, q); what is left splits the channels."""
    if world < 1:
        raise ValueError("world must be >= 1")
    wb = math.gcd(B, world) if B > 0 else 1
    wm = world // wb
    if wm > max(M, 1):
        raise ValueError(f"cannot split B={B}, M={M} over {world} ranks")
    return wb, wm


def block_of(B: int, M: int, world: int, rank: int, align: int = 32) -> Block:
    """Block of rank ``rank``. Channel blocks are contiguous, multiples of
    ``align`` channels where M allows (a CTA covers 32 channels), and differ in
    size by at most one ``align`` unit."""
    wb, wm = grid_for(B, M, world, align)
    br, cr = rank // wm, rank % wm
    per_b = B // wb
    b0, b1 = br * per_b, (br + 1) * per_b
    unit = align if M % align == 0 and M // align >= wm else 1
    units = M // unit
    base, extra = divmod(units, wm)
    m0 = (cr * base + min(cr, extra)) * unit
    m1 = m0 + (base + (1 if cr < extra else 0)) * unit
    return Block(b0, b1, m0, m1, br, cr, wb, wm)


class Groups(NamedTuple):
    batch_group: Optional[dist.ProcessGroup]    # same channels, different batch elements
    channel_group: Optional[dist.ProcessGroup]  # same batch elements, different channels


def make_groups(world: int, wb: int, wm: int) -> Groups:
    """Create the two families of process groups (every rank must call this with
    the same arguments; ``dist.new_group`` is collective)."""
    rank = dist.get_rank()
    batch_group = channel_group = None
    if wb > 1:
        for cr in range(wm):
            g = dist.new_group([br * wm + cr for br in range(wb)])
            if rank % wm == cr:
                batch_group = g
    if wm > 1:
        for br in range(wb):
            g = dist.new_group([br * wm + cr for cr in range(wm)])
            if rank // wm == br:
                channel_group = g
    return Groups(batch_group, channel_group)


class _SumGradOver(torch.autograd.Function):
    """Identity in the forward; all-reduce (sum) of the gradient in the backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, op=dist.ReduceOp.SUM, group=ctx.group)
        return g, None


def sum_grad_over(x: torch.Tensor, group) -> torch.Tensor:
    return x if group is None else _SumGradOver.apply(x, group)


class _SumGradsOver(torch.autograd.Function):
    """Identity on several tensors in the forward; ONE all-reduce (sum) of all their gradients in the backward:
    the gradients are small here, so a step pays per collective call, not per byte."""

    @staticmethod
    def forward(ctx, group, *xs):
        ctx.group = group
        return tuple(x.view_as(x) for x in xs)

    @staticmethod
    def backward(ctx, *gs):
        live = [g for g in gs if g is not None]
        if not live:
            return (None, *gs)
        flat = torch.cat([g.reshape(-1).to(live[0].dtype) for g in live])
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=ctx.group)
        parts = iter(flat.split([g.numel() for g in live]))
        return (None, *[None if g is None else next(parts).view_as(g).to(g.dtype) for g in gs])


def sum_grads_over(xs, group):
    """``sum_grad_over`` for several tensors at once, with a single collective."""
    return tuple(xs) if group is None else _SumGradsOver.apply(group, *xs)


def take_block(blk: Block, v, lambda_v, k, q, a, p, initial_state=None):
    """Slice full tensors down to one rank's block (views, no copies)."""
    bs, ms = slice(blk.b0, blk.b1), slice(blk.m0, blk.m1)
    st = None
    if initial_state is not None:
        st = (initial_state[0][bs, ms], initial_state[1][bs, ms])
    return v[bs, :, ms], lambda_v[bs, :, ms], k[bs], q[bs], a[ms], p[ms], st


def scan_block(scan_fn: Callable, groups: Groups, v, lambda_v, k, q, a, p,
               initial_state=None, decode_from_prior: bool = False):
    """Scan this rank's block with ``scan_fn`` (e.g. ``kla_scan_b200``). The
    forward communicates nothing; in the backward the gradients of a, p are
    summed over the batch group and those of k, q over the channel group, so
    every rank ends with the gradients of the full problem for its slices (one collective per group)."""
    a, p = sum_grads_over((a, p), groups.batch_group)
    k, q = sum_grads_over((k, q), groups.channel_group)
    return scan_fn(v, lambda_v, k, q, a, p, initial_state=initial_state,
                   decode_from_prior=decode_from_prior)
