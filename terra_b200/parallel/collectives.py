"""Autograd-aware collectives on ``torch.distributed`` groups (gloo on CPU, NCCL on GPU).

These are the portable building blocks of the multi-rank layouts and the baseline that the fused peer-memory
kernels are measured against. Only primitives that gloo implements are used in the CPU branches
(all_gather on lists, all_reduce, send/recv), so every multi-rank code path can be exercised without a GPU.

Gradient conventions (the loss of the job is the SUM of the per-rank losses):
  all-gather        <->  reduce-scatter (sum)
  reduce-scatter    <->  all-gather
  all-reduce (sum)  <->  all-reduce (sum)
  halo exchange     <->  halo gradients travel back and are added to the rows they were copied from
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


def _is_nccl(group) -> bool:
    try:
        return dist.get_backend(group) == "nccl"
    except Exception:
        return False


def group_size(group) -> int:
    return dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1


def group_rank(group) -> int:
    return dist.get_rank(group) if (dist.is_available() and dist.is_initialized()) else 0


def _gather_ragged(x: torch.Tensor, group, sizes: Sequence[int]) -> torch.Tensor:
    """Concatenate every rank's ``x`` (dim 0 extents ``sizes``) in group-rank order."""
    world = len(sizes)
    mx = max(sizes)
    pad = x
    if x.shape[0] != mx:
        pad = x.new_zeros((mx,) + tuple(x.shape[1:]))
        pad[:x.shape[0]] = x
    pad = pad.contiguous()
    if _is_nccl(group):
        out = x.new_empty((world * mx,) + tuple(x.shape[1:]))
        dist.all_gather_into_tensor(out, pad, group=group)
        parts = list(out.split(mx, dim=0))
    else:
        parts = [torch.empty_like(pad) for _ in range(world)]
        dist.all_gather(parts, pad, group=group)
    return torch.cat([p[:n] for p, n in zip(parts, sizes)], dim=0)


def _reduce_scatter_ragged(x: torch.Tensor, group, sizes: Sequence[int]) -> torch.Tensor:
    """Sum ``x`` over the group and return this rank's dim-0 slice."""
    r = dist.get_rank(group)
    start = sum(sizes[:r])
    if _is_nccl(group) and len(set(sizes)) == 1:
        out = x.new_empty((sizes[r],) + tuple(x.shape[1:]))
        dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
        return out
    full = x.contiguous().clone()
    dist.all_reduce(full, group=group)
    return full[start:start + sizes[r]].contiguous()


class _AllGatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, sizes):
        ctx.group, ctx.sizes = group, tuple(sizes)
        return _gather_ragged(x, group, sizes)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter_ragged(g, ctx.group, ctx.sizes), None, None


class _ReduceScatterRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, sizes):
        ctx.group, ctx.sizes = group, tuple(sizes)
        return _reduce_scatter_ragged(x, group, sizes)

    @staticmethod
    def backward(ctx, g):
        return _gather_ragged(g, ctx.group, ctx.sizes), None, None


class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        y = x.contiguous().clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        gg = g.contiguous().clone()
        dist.all_reduce(gg, group=ctx.group)
        return gg, None


def all_gather_rows(x, group, sizes: Optional[Sequence[int]] = None):
    world = group_size(group)
    if world == 1:
        return x
    return _AllGatherRows.apply(x, group, list(sizes) if sizes is not None else [x.shape[0]] * world)


def reduce_scatter_rows(x, group, sizes: Optional[Sequence[int]] = None):
    world = group_size(group)
    if world == 1:
        return x
    return _ReduceScatterRows.apply(x, group, list(sizes) if sizes is not None else [x.shape[0] // world] * world)


def all_reduce_sum(x, group):
    if group_size(group) == 1:
        return x
    return _AllReduceSum.apply(x, group)


def all_reduce_(x: torch.Tensor, group) -> torch.Tensor:
    """In-place, no autograd (gradient buckets, statistics)."""
    if group_size(group) > 1:
        dist.all_reduce(x, group=group)
    return x


def _exchange(send_prev, send_next, prev_rank, next_rank, group):
    """Send one tensor to each neighbour and receive one from each; ``None`` rank = no neighbour."""
    recv_prev = torch.empty_like(send_next) if prev_rank is not None else None
    recv_next = torch.empty_like(send_prev) if next_rank is not None else None
    ops = []
    if prev_rank is not None:
        ops.append(dist.P2POp(dist.isend, send_prev.contiguous(), prev_rank, group))
        ops.append(dist.P2POp(dist.irecv, recv_prev, prev_rank, group))
    if next_rank is not None:
        ops.append(dist.P2POp(dist.isend, send_next.contiguous(), next_rank, group))
        ops.append(dist.P2POp(dist.irecv, recv_next, next_rank, group))
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    return recv_prev, recv_next


class _HaloRows(torch.autograd.Function):
    """x: [B, C, H, W] row stripe -> [B, C, H + 2*halo, W] with neighbour rows, zeros at the global edges
    (non-periodic; reference: credit/domain_parallel/halo_exchange.py:18-157)."""

    @staticmethod
    def forward(ctx, x, halo, prev_rank, next_rank, group):
        ctx.p = (halo, prev_rank, next_rank, group)
        top_rows = x[:, :, :halo].contiguous()
        bot_rows = x[:, :, -halo:].contiguous()
        recv_prev, recv_next = _exchange(top_rows, bot_rows, prev_rank, next_rank, group)
        top = recv_prev if recv_prev is not None else torch.zeros_like(top_rows)
        bot = recv_next if recv_next is not None else torch.zeros_like(bot_rows)
        return torch.cat([top, x, bot], dim=2)

    @staticmethod
    def backward(ctx, g):
        halo, prev_rank, next_rank, group = ctx.p
        g_top = g[:, :, :halo].contiguous()        # gradient of rows that belong to prev
        g_bot = g[:, :, -halo:].contiguous()       # gradient of rows that belong to next
        gx = g[:, :, halo:-halo].clone()
        from_prev, from_next = _exchange(g_top, g_bot, prev_rank, next_rank, group)
        # prev sent me the gradient of my top rows (it held them as its bottom halo), next likewise
        if from_prev is not None:
            gx[:, :, :halo] += from_prev
        if from_next is not None:
            gx[:, :, -halo:] += from_next
        return gx, None, None, None, None


def halo_rows(x, halo: int, prev_rank, next_rank, group):
    return _HaloRows.apply(x, halo, prev_rank, next_rank, group)
