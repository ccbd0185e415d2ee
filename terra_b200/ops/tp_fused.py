"""Tensor-parallel linear layers with the collective fused into the GEMM over NVLink peer memory.

* ``ag_gemm``: all-gather -> GEMM. Every rank leaves its ``[rows, K]`` activation shard in symmetric memory; the
  tcgen05 GEMM reads the concatenation tile by tile with one TMA tensor map per peer (plain peer loads, no cluster
  fan-out), its own shard's tiles first, so the NVLink transfers overlap the math of the tiles already resident.
  Nothing of size ``[M, K]`` is materialised.
* ``gemm_rs``: GEMM -> reduce-scatter. The rank's partial product over its slice of K is reduced from the epilogue
  straight into the fp32 accumulation buffer of each row block's owner (16-byte vector reductions over NVLink).
* ``TpMlp``: the MLP half of a transformer block on sequence-sharded activations with column / row sharded
  weights, forward and backward built from those two primitives (the backward of one is the other).

The reference reaches the same result with ``all_gather_into_tensor`` / ``reduce_scatter_tensor`` calls around cuBLAS
GEMMs (models/parallel_layers.py, the TP branches of the MLP)."""
from __future__ import annotations

from typing import Optional

import torch

from .gemm import gemm


class TpFusedComm:
    """Symmetric staging for the fused TP linears of one tensor-parallel group (``arena``: a SymmetricArena over it)."""

    def __init__(self, arena):
        self.arena = arena
        self.rank, self.world = arena.rank, arena.world

    # ---- all-gather -> GEMM
    def stage(self, x: torch.Tensor) -> torch.Tensor:
        """Copy this rank's shard into symmetric memory (unless it already lives there) and publish it."""
        try:
            self.arena.offset_of(x)
            staged = x
        except ValueError:
            staged = self.arena.alloc(tuple(x.shape), x.dtype)
            staged.copy_(x)
        self.arena.barrier()            # every rank's shard is complete before anybody's GEMM reads it
        return staged

    def ag_gemm(self, x_shard: torch.Tensor, w: torch.Tensor, *, b_mn: bool = False, bias=None, gelu=False,
                save_pre=False, dgelu_aux=None, release: bool = True):
        """``concat_ranks(x_shard) @ w^T`` (or ``@ w`` with ``b_mn``) with the usual fused epilogues. ``release`` ends
        with a barrier after which the staged shards may be overwritten."""
        staged = self.stage(x_shard)
        out = gemm(staged, w, b_mn=b_mn, bias=bias, gelu=gelu, save_pre=save_pre, dgelu_aux=dgelu_aux,
                   a_peers=self.arena.peer_ptrs(staged), rank=self.rank)
        if release:
            self.arena.barrier()
        return out

    # ---- GEMM -> reduce-scatter
    def gemm_rs(self, a: torch.Tensor, w: torch.Tensor, *, b_mn: bool = False) -> torch.Tensor:
        """Row block ``rank`` of ``sum_ranks(a @ w^T)`` as fp32 ``[M / world, N]`` (a view into symmetric memory, valid
        until the arena is reset)."""
        M = a.shape[0]
        N = w.shape[1] if b_mn else w.shape[0]
        if M % self.world:
            raise ValueError(f"{M} rows cannot be scattered over {self.world} ranks")
        acc = self.arena.alloc((M // self.world, N), torch.float32)
        acc.zero_()
        self.arena.barrier()            # all accumulation buffers are zero before the first reduction arrives
        gemm(a, w, b_mn=b_mn, out=acc, out_peers=self.arena.peer_ptrs(acc), rank=self.rank)
        self.arena.barrier()            # all partial products have landed
        return acc


class _TpMlpFn(torch.autograd.Function):
    """y_shard = x_shard + fc2(gelu(fc1(LN(x)))) with x sequence-sharded over the TP group, fc1 column-sharded
    ([F / tp, C]) and fc2 row-sharded ([C, F / tp]); ``xn`` is the already normalised shard."""

    @staticmethod
    def forward(ctx, xn, w1, b1, w2, comm: TpFusedComm):
        act, pre = comm.ag_gemm(xn, w1, bias=b1, gelu=True, save_pre=True)          # [M, F/tp]
        y = comm.gemm_rs(act, w2)                                                      # fp32 [M/tp, C]
        ctx.save_for_backward(xn, w1, w2, pre, act)
        ctx.comm = comm
        return y.to(torch.bfloat16)

    @staticmethod
    def backward(ctx, dy):
        xn, w1, w2, pre, act = ctx.saved_tensors
        comm: TpFusedComm = ctx.comm
        dy = dy.contiguous().to(torch.bfloat16)
        staged_dy = comm.stage(dy)
        # d(act) = gather(dy) @ w2, times GELU'(pre): all-gather -> GEMM again (the backward of the reduce-scatter)
        dpre = gemm(staged_dy, w2, b_mn=True, dgelu_aux=pre, a_peers=comm.arena.peer_ptrs(staged_dy), rank=comm.rank)
        # weight gradients need the gathered operands once; plain peer copies, off the critical path of dgrad
        dy_full = _gather_rows(comm, staged_dy)
        comm.arena.barrier()
        gw2 = gemm(dy_full, act, a_mn=True, b_mn=True, out_f32=True, accumulate=True, split_k=_wgrad_split(dy_full, act))
        staged_xn = comm.stage(xn)
        xn_full = _gather_rows(comm, staged_xn)
        comm.arena.barrier()
        gw1 = gemm(dpre, xn_full, a_mn=True, b_mn=True, out_f32=True, accumulate=True, split_k=_wgrad_split(dpre, xn_full))
        gb1 = dpre.float().sum(0)
        # d(xn) = reduce-scatter(dpre @ w1): GEMM -> reduce-scatter (the backward of the all-gather)
        dxn = comm.gemm_rs(dpre, w1, b_mn=True)
        return dxn.to(torch.bfloat16), gw1.to(w1.dtype), gb1.to(w1.dtype), gw2.to(w2.dtype), None


def _wgrad_split(a, b) -> int:
    tiles = ((a.shape[1] + 127) // 128) * ((b.shape[1] + 127) // 128)
    return max(1, min((a.shape[0] + 63) // 64, 148 // max(1, tiles)))


def _gather_rows(comm: TpFusedComm, staged: torch.Tensor) -> torch.Tensor:
    """Concatenation of every rank's staged shard by peer-to-peer row copies (used for the weight gradients)."""
    from .. import _ext

    ext = _ext.load()
    rows, cols = staged.shape
    full = torch.empty(rows * comm.world, cols, dtype=staged.dtype, device=staged.device)
    nbytes = cols * staged.element_size()
    for r, ptr in enumerate(comm.arena.peer_ptrs(staged)):
        ext.peer_copy_rows(full[r * rows:(r + 1) * rows].data_ptr(), ptr, rows, nbytes, nbytes, nbytes)
    return full


def tp_mlp(xn: torch.Tensor, w1: torch.Tensor, b1: Optional[torch.Tensor], w2: torch.Tensor, comm: TpFusedComm):
    """Sequence-sharded MLP body (without the residual and fc2's bias, which the caller adds once)."""
    return _TpMlpFn.apply(xn, w1, b1, w2, comm)
