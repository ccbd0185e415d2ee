"""Autograd-aware collectives on ``torch.distributed`` groups (gloo on CPU, NCCL on GPU).

These are the portable building blocks of the multi-rank layouts and the baseline that the fused peer-memory
kernels are measured against. Only primitives that gloo implements are used in the CPU branches
(all_gather on lists, all_reduce, all_to_all_single, send/recv), so every multi-rank code path can be exercised without a GPU.

Gradient conventions (the loss of the job is the SUM of the per-rank losses):
  all-gather        <->  reduce-scatter (sum)
  reduce-scatter    <->  all-gather
  all-reduce (sum)  <->  all-reduce (sum)
  all-to-all        <->  all-to-all with the chunk extents swapped
  ring transfer     <->  ring transfer in the opposite direction
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


class _AllToAllRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, send_sizes, recv_sizes):
        ctx.group, ctx.send_sizes, ctx.recv_sizes = group, send_sizes, recv_sizes
        x = x.contiguous()
        out = x.new_empty((sum(recv_sizes),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x, output_split_sizes=list(recv_sizes), input_split_sizes=list(send_sizes), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        # the adjoint sends every received chunk's gradient back where the chunk came from
        return _AllToAllRows.apply(g.contiguous(), ctx.group, ctx.recv_sizes, ctx.send_sizes), None, None, None


def all_to_all_rows(x, group, send_sizes: Optional[Sequence[int]] = None, recv_sizes: Optional[Sequence[int]] = None):
    """The rows of ``x``, cut into one consecutive chunk per group rank (extents ``send_sizes``), travel to their rank;
    returns the chunks received from every rank, concatenated in group-rank order (extents ``recv_sizes``). Defaults:
    equal chunks. The Ulysses exchange of the sequence-parallel baseline and the all-to-all-v of a general relayout
    (reference: core/tensor_parallel.py:291-356, core/parallel/layout_transform.py:107-173)."""
    world = group_size(group)
    if world == 1:
        return x
    if send_sizes is None:
        if x.shape[0] % world:
            raise ValueError(f"all_to_all_rows: {x.shape[0]} rows do not split evenly over {world} ranks")
        send_sizes = [x.shape[0] // world] * world
    if recv_sizes is None:
        recv_sizes = list(send_sizes)
    if sum(send_sizes) != x.shape[0] or len(send_sizes) != world or len(recv_sizes) != world:
        raise ValueError("all_to_all_rows: chunk extents do not match the tensor / the group")
    return _AllToAllRows.apply(x, group, list(send_sizes), list(recv_sizes))


class _RingTransfer(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, shift):
        ctx.group, ctx.shift = group, shift
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        dst = dist.get_global_rank(group, (rank + shift) % world)
        src = dist.get_global_rank(group, (rank - shift) % world)
        x = x.contiguous()
        out = torch.empty_like(x)
        reqs = dist.batch_isend_irecv([dist.P2POp(dist.isend, x, dst, group), dist.P2POp(dist.irecv, out, src, group)])
        for r in reqs:
            r.wait()
        return out

    @staticmethod
    def backward(ctx, g):
        return _RingTransfer.apply(g.contiguous(), ctx.group, -ctx.shift), None, None


def ring_transfer(x, group, shift: int = 1):
    """Every rank sends ``x`` to the rank ``shift`` places further along the group's ring and returns what it receives
    from the rank ``shift`` places behind (same shape on every rank). Gradients travel the ring the other way
    (reference: core/p2p_comm.py:4-71, the +-1 ring of the regular window-parallel shift)."""
    world = group_size(group)
    if world == 1 or shift % world == 0:
        return x
    return _RingTransfer.apply(x, group, int(shift))


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
