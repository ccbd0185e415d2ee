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

from ..parallel.nvlink import BARRIER_SPIN_LIMIT as PEER_WAIT_NS
from .. import _ext
from .gemm import gemm


class TpFusedComm:
    """Symmetric staging for the fused TP linears of one tensor-parallel group (``arena``: a SymmetricArena over it)."""

    def __init__(self, arena):
        self.arena = arena
        self.rank, self.world = arena.rank, arena.world
        self.side: Optional[torch.cuda.Stream] = None   # stream of the copy-engine gather

    # ---- all-gather -> GEMM
    def stage(self, x: torch.Tensor) -> torch.Tensor:
        """This rank's shard in symmetric memory (copied there unless it already is)."""
        try:
            self.arena.offset_of(x)
            return x
        except ValueError:
            staged = self.arena.alloc(tuple(x.shape), x.dtype)
            staged.copy_(x)
            return staged

    def ag_gemm(self, x_shard: torch.Tensor, w: torch.Tensor, *, b_mn: bool = False, bias=None, gelu=False,
                save_pre=False, dgelu_aux=None, via_copy_engine: Optional[bool] = None):
        """``concat_ranks(x_shard) @ w^T`` (or ``@ w`` with ``b_mn``) with the usual fused epilogues. No barrier in
        front: every rank publishes its shard with a one-way signal and the GEMM's TMA thread waits (bounded) for
        what it needs right before its first tile of a peer's rows, while the tiles of the own shard are computing.

        Two transports. Direct: the GEMM's TMA loads read the peers' shards over NVLink - every output column tile
        fetches its A tiles again (a peer's memory is not cached in the local L2), so this is for outputs of one
        column tile (N <= 256). Copy engine (default for wider outputs): a side stream waits for each peer's signal
        with a stream memory operation, copies the shard into local memory with the copy engines and publishes
        "ready" with another stream memory operation, all without an SM (a kernel could not be scheduled beside the
        persistent GEMM); the GEMM reads local memory and waits on the ready words. The shard crosses NVLink once.
        The staged shards stay untouched until the next barrier of the group (``gemm_rs`` ends with one)."""
        staged = self.stage(x_shard)
        epoch = self.arena.publish()
        N = w.shape[1] if b_mn else w.shape[0]
        if via_copy_engine is None:
            via_copy_engine = N > 256
        kw = dict(b_mn=b_mn, bias=bias, gelu=gelu, save_pre=save_pre, dgelu_aux=dgelu_aux, rank=self.rank, a_epoch=epoch,
                  a_budget_ns=PEER_WAIT_NS)
        if not via_copy_engine:
            return gemm(staged, w, a_peers=self.arena.peer_ptrs(staged), a_flags=self.arena.signal_flags_ptr, **kw)
        rows, K = staged.shape
        gathered = torch.empty(self.world * rows, K, dtype=staged.dtype, device=staged.device)
        main = torch.cuda.current_stream(staged.device)
        if self.side is None:
            self.side = torch.cuda.Stream(staged.device)
        gathered.record_stream(self.side)
        self.side.wait_stream(main)                     # `gathered` exists, earlier users of the ready words are queued
        row_bytes = K * staged.element_size()
        nbytes = rows * row_bytes
        # up to four pieces per peer, each a whole number of 128-row tiles: the GEMM starts on a peer's rows as soon
        # as their piece has landed
        tiles = (rows + 127) // 128
        chunks = max(1, min(4, tiles))
        chunk_tiles = (tiles + chunks - 1) // chunks
        _ext.load().gather_shards_async(self.side.cuda_stream, gathered.data_ptr(), self.arena.peer_ptrs(staged),
                                        self.rank, rows, row_bytes, chunks, chunk_tiles * 128,
                                        self.arena.signal_flags_ptr, self.arena.ready_flags_ptr, epoch)
        local = [gathered.data_ptr() + r * nbytes for r in range(self.world)]
        local[self.rank] = staged.data_ptr()            # the own shard is read in place
        out = gemm(staged, w, a_peers=local, a_flags=self.arena.ready_flags_ptr, a_interleave=False, a_chunks=chunks, **kw)
        main.wait_stream(self.side)                     # the peers' shards have been read before this rank's next barrier
        return out

    # ---- GEMM -> reduce-scatter
    def gemm_rs(self, a: torch.Tensor, w: torch.Tensor, *, b_mn: bool = False, exact: bool = False) -> torch.Tensor:
        """Row block ``rank`` of ``sum_ranks(a @ w^T)``: ``[M / world, N]``, bf16 (fp32 with ``exact``).

        Default: every rank stores its bf16 partial of row block j into its own slot of owner j's staging (plain
        16-byte stores over NVLink, no zeroing, no atomics); after one barrier the owner adds the slots up in fp32.
        ``exact``: fp32 vector reductions into the owner's accumulation buffer instead (twice the NVLink bytes and a
        zero + barrier in front, but the partials are not rounded to bf16)."""
        M = a.shape[0]
        N = w.shape[1] if b_mn else w.shape[0]
        if M % self.world:
            raise ValueError(f"{M} rows cannot be scattered over {self.world} ranks")
        rows = M // self.world
        if exact:
            acc = self.arena.alloc((rows, N), torch.float32)
            acc.zero_()
            self.arena.barrier()        # all accumulation buffers are zero before the first reduction arrives
            gemm(a, w, b_mn=b_mn, out=acc, out_peers=self.arena.peer_ptrs(acc), rank=self.rank)
            self.arena.barrier()        # all partial products have landed
            return acc
        slots = self.arena.alloc((self.world, rows, N), torch.bfloat16)
        gemm(a, w, b_mn=b_mn, out=slots, out_peers=self.arena.peer_ptrs(slots), rank=self.rank)
        self.arena.barrier()            # every rank's partial has landed in this rank's slots
        out = torch.empty(rows, N, dtype=torch.bfloat16, device=a.device)
        _ext.load().sum_slots(slots, out)
        return out


class _TpMlpFn(torch.autograd.Function):
    """y_shard = fc2(gelu(fc1(xn))) with xn (the normalised activations) sequence-sharded over the TP group, fc1
    column-sharded ([F / tp, C]) and fc2 row-sharded ([C, F / tp]). ``grads`` = (gw1, gb1, gw2): fp32 buffers of the
    flat parameter arena that the weight gradients are accumulated into (then ``anchor``, any parameter, keeps the
    node in the graph and no parameter gradient is returned); ``None``: the gradients are returned."""

    @staticmethod
    def forward(ctx, xn, anchor, w1, b1, w2, grads, comm: TpFusedComm):
        act, pre = comm.ag_gemm(xn, w1, bias=b1, gelu=True, save_pre=True)          # [M, F/tp]
        y = comm.gemm_rs(act, w2)                                                      # fp32 [M/tp, C]
        ctx.save_for_backward(xn, w1, w2, pre, act)
        ctx.comm, ctx.grads = comm, grads
        return y.to(torch.bfloat16)

    @staticmethod
    def backward(ctx, dy):
        from .blocks import bias_grad_accumulate, wgrad_accumulate

        xn, w1, w2, pre, act = ctx.saved_tensors
        comm: TpFusedComm = ctx.comm
        dy = dy.contiguous().to(torch.bfloat16)
        staged_dy, staged_xn = comm.stage(dy), comm.stage(xn)
        # d(act) = gather(dy) @ w2, times GELU'(pre): all-gather -> GEMM again (the backward of the reduce-scatter)
        dpre = comm.ag_gemm(staged_dy, w2, b_mn=True, dgelu_aux=pre)
        # weight gradients need the gathered operands once: plain peer copies after a barrier (it also covers xn)
        comm.arena.barrier()
        dy_full = _gather_rows(comm, staged_dy)
        xn_full = _gather_rows(comm, staged_xn)
        if ctx.grads is not None:
            gw1, gb1, gw2 = ctx.grads
            wgrad_accumulate(dy_full, act, gw2)
            wgrad_accumulate(dpre, xn_full, gw1)
            if gb1 is not None:
                bias_grad_accumulate(dpre, gb1)
            ret = (None, None, None)
        else:
            gw2 = gemm(dy_full, act, a_mn=True, b_mn=True, out_f32=True, accumulate=True, split_k=_wgrad_split(dy_full, act))
            gw1 = gemm(dpre, xn_full, a_mn=True, b_mn=True, out_f32=True, accumulate=True, split_k=_wgrad_split(dpre, xn_full))
            ret = (gw1.to(w1.dtype), dpre.float().sum(0).to(w1.dtype), gw2.to(w2.dtype))
        # d(xn) = reduce-scatter(dpre @ w1): GEMM -> reduce-scatter (the backward of the all-gather)
        dxn = comm.gemm_rs(dpre, w1, b_mn=True)
        return dxn.to(torch.bfloat16), None, ret[0], ret[1], ret[2], None, None


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


def tp_mlp(xn: torch.Tensor, w1: torch.Tensor, b1: Optional[torch.Tensor], w2: torch.Tensor, comm: TpFusedComm,
           anchor: Optional[torch.Tensor] = None, grads=None):
    """Sequence-sharded MLP body (without the residual and fc2's bias, which the caller adds once)."""
    return _TpMlpFn.apply(xn, anchor, w1, b1, w2, grads, comm)
