"""Tensor- and sequence-parallel building blocks in their classic forms, on autograd-aware collectives
(capabilities of the reference's core/tensor_parallel.py:10-610 and of the MLP variants built on it, models/mlp.py:177-373).

Region functions (the collective sits on one side of the autograd graph, its adjoint on the other):

  ``copy_to_region``         identity forward, all-reduce backward      (input of a column-parallel layer)
  ``reduce_from_region``     all-reduce forward, identity backward      (output of a row-parallel layer)
  ``gather_from_region``     all-gather of the last dimension forward, this rank's slice of the gradient backward
  ``scatter_to_region``      this rank's slice of the last dimension forward, all-gather of the gradient backward
  ``all_gather_dim``         all-gather along any dimension forward, reduce-scatter backward   (sequence parallel in)
  ``reduce_scatter_dim``     reduce-scatter along any dimension forward, all-gather backward   (sequence parallel out)
  ``all_to_all_dims``        cut ``split_dim`` over the ranks and concatenate what arrives along ``concat_dim``
                             (Ulysses head <-> token exchange); its adjoint swaps the two dimensions

and three MLP layers over a model-parallel group: ``TensorParallelMLP`` (Megatron: column-parallel fc1, row-parallel fc2,
one all-reduce each way), ``MegatronSequenceParallelMLP`` (activations sharded along the tokens outside the layer:
all-gather in, reduce-scatter out) and ``UlyssesSequenceParallelMLP`` (token shards, replicated weights, no
communication; parameter gradients are summed by the caller's gradient reduction).

The model of this repository runs its tensor-parallel halves on the fused all-gather / reduce-scatter GEMM kernels
(``ops/tp_fused.py``); these classes are the portable forms, and the Megatron all-reduce variant the fused kernels do
not cover.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from . import collectives as C


def ensure_divisibility(numerator: int, denominator: int) -> None:
    if numerator % denominator != 0:
        raise ValueError(f"{numerator} is not divisible by {denominator}")


def divide(numerator: int, denominator: int) -> int:
    ensure_divisibility(numerator, denominator)
    return numerator // denominator


def split_tensor_along_last_dim(tensor: torch.Tensor, num_partitions: int, contiguous_split_chunks: bool = False):
    chunks = torch.split(tensor, divide(tensor.shape[-1], num_partitions), dim=-1)
    return tuple(c.contiguous() for c in chunks) if contiguous_split_chunks else chunks


class _CopyToRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


def copy_to_region(x, group):
    return x if C.group_size(group) == 1 else _CopyToRegion.apply(x, group)


class _ReduceFromRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        y = x.contiguous().clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None


def reduce_from_region(x, group):
    return x if C.group_size(group) == 1 else _ReduceFromRegion.apply(x, group)


def all_gather_dim(x, dim: int, group):
    """Concatenate every rank's ``x`` along ``dim``; the gradient is reduce-scattered back."""
    if C.group_size(group) == 1:
        return x
    dim = dim % x.ndim
    return C.all_gather_rows(x.movedim(dim, 0).contiguous(), group).movedim(0, dim)


def reduce_scatter_dim(x, dim: int, group):
    """Sum over the ranks, each keeping its equal share along ``dim``; the gradient is all-gathered back."""
    if C.group_size(group) == 1:
        return x
    dim = dim % x.ndim
    ensure_divisibility(x.shape[dim], C.group_size(group))
    return C.reduce_scatter_rows(x.movedim(dim, 0).contiguous(), group).movedim(0, dim)


class _SliceLastDim(torch.autograd.Function):
    """This rank's slice of the last dimension; the gradient slices of all ranks are gathered back."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n, r = dist.get_world_size(group), dist.get_rank(group)
        return split_tensor_along_last_dim(x, n)[r].contiguous()

    @staticmethod
    def backward(ctx, g):
        parts = [torch.empty_like(g) for _ in range(dist.get_world_size(ctx.group))]
        dist.all_gather(parts, g.contiguous(), group=ctx.group)
        return torch.cat(parts, dim=-1), None


class _GatherLastDim(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        parts = [torch.empty_like(x) for _ in range(dist.get_world_size(group))]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, dim=-1)

    @staticmethod
    def backward(ctx, g):
        n, r = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
        return split_tensor_along_last_dim(g, n)[r].contiguous(), None


def scatter_to_region(x, group):
    return x if C.group_size(group) == 1 else _SliceLastDim.apply(x, group)


def gather_from_region(x, group):
    return x if C.group_size(group) == 1 else _GatherLastDim.apply(x, group)


def all_to_all_dims(x, group, split_dim: int, concat_dim: int):
    """Cut ``split_dim`` into one equal chunk per rank, send chunk ``j`` to rank ``j``, concatenate the chunks received
    (in rank order) along ``concat_dim``: ``[..., S / n, ..., H, ...] -> [..., S, ..., H / n, ...]`` for the Ulysses
    exchange. Differentiable (the adjoint is the same call with the two dimensions swapped)."""
    n = C.group_size(group)
    if n == 1:
        return x
    split_dim, concat_dim = split_dim % x.ndim, concat_dim % x.ndim
    ensure_divisibility(x.shape[split_dim], n)
    # rows of the exchange = (destination rank, everything else)
    chunks = x.reshape(*x.shape[:split_dim], n, x.shape[split_dim] // n, *x.shape[split_dim + 1:]).movedim(split_dim, 0)
    rest = tuple(chunks.shape[1:])                                 # shape of one chunk
    flat = chunks.contiguous().reshape(n * rest[0], *rest[1:])     # rows grouped by destination rank
    got = C.all_to_all_rows(flat, group).reshape(n, *rest)         # [source rank, ...chunk shape...]
    # the source-rank axis becomes the outer factor of concat_dim
    shape = list(rest)
    shape[concat_dim] *= n
    return got.movedim(0, concat_dim).reshape(*shape)


def generic_all_to_all_group(x, group, group_size, split_dim, concat_dim):
    """Call-compatible with the reference's helper of this name (``group_size`` is implied by ``group``)."""
    return all_to_all_dims(x, group, split_dim, concat_dim)


# ------------------------------------------------------------------------------------------------ layers
def _shard_linear(fin: int, fout: int, rank: int, n: int, split_rows: bool):
    """This rank's part of a freshly initialised ``nn.Linear(fin, fout)``: rows ``[out / n, in]`` with the matching bias
    slice (column-parallel layer), or columns ``[out, in / n]`` with the whole bias (row-parallel layer). Every rank
    draws the same full layer from the current RNG state and keeps its part."""
    full = nn.Linear(fin, fout)
    if split_rows:
        per = divide(fout, n)
        return (nn.Parameter(full.weight.detach()[rank * per:(rank + 1) * per].clone()),
                nn.Parameter(full.bias.detach()[rank * per:(rank + 1) * per].clone()))
    per = divide(fin, n)
    return nn.Parameter(full.weight.detach()[:, rank * per:(rank + 1) * per].clone()), nn.Parameter(full.bias.detach().clone())


class TensorParallelMLP(nn.Module):
    """``x + fc2(gelu(fc1(norm(x))))`` with fc1 column-parallel and fc2 row-parallel over ``group`` (Megatron): the
    activations are replicated, one all-reduce of the output forward and one of the input gradient backward."""

    def __init__(self, group, in_features: int, hidden_features: int, out_features: Optional[int] = None,
                 use_layernorm: bool = True):
        super().__init__()
        out_features = out_features or in_features
        self.group = group
        n, r = C.group_size(group), C.group_rank(group)
        self.norm2 = nn.LayerNorm(in_features) if use_layernorm else nn.Identity()
        self.weight1, self.bias1 = _shard_linear(in_features, hidden_features, r, n, split_rows=True)
        self.weight2, self.bias2 = _shard_linear(hidden_features, out_features, r, n, split_rows=False)

    def forward(self, x):
        h = copy_to_region(self.norm2(x), self.group)
        h = F.gelu(F.linear(h, self.weight1, self.bias1))
        y = reduce_from_region(F.linear(h, self.weight2), self.group)
        return x + y + self.bias2.to(y.dtype)


class MegatronSequenceParallelMLP(TensorParallelMLP):
    """The same weights with the activations sharded along ``seq_dim`` outside the layer: all-gather of the normalised
    shard in, reduce-scatter of the partial outputs out (the norm and the residual work on the shard)."""

    def __init__(self, group, in_features: int, hidden_features: int, out_features: Optional[int] = None,
                 use_layernorm: bool = True, seq_dim: int = 1):
        super().__init__(group, in_features, hidden_features, out_features, use_layernorm)
        self.seq_dim = seq_dim

    def forward(self, x):
        h = all_gather_dim(self.norm2(x), self.seq_dim, self.group)
        h = F.gelu(F.linear(h, self.weight1, self.bias1))
        y = reduce_scatter_dim(F.linear(h, self.weight2), self.seq_dim, self.group)
        return x + y + self.bias2.to(y.dtype)


class UlyssesSequenceParallelMLP(nn.Module):
    """Token shards through a replicated MLP: no communication in the layer; the parameter gradients of the ranks are
    partial sums over their tokens and are added by the job's gradient reduction."""

    def __init__(self, in_features: int, hidden_features: int, out_features: Optional[int] = None, use_layernorm: bool = True):
        super().__init__()
        self.norm2 = nn.LayerNorm(in_features) if use_layernorm else nn.Identity()
        self.fc1 = nn.Linear(in_features, hidden_features)
        self.fc2 = nn.Linear(hidden_features, out_features or in_features)

    def forward(self, x):
        return x + self.fc2(F.gelu(self.fc1(self.norm2(x))))
