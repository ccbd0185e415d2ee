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
from .packed import fp32_values


class TpFusedComm:
    """Symmetric staging for the fused TP linears of one tensor-parallel group (``arena``: a SymmetricArena over it)."""

    def __init__(self, arena):
        self.arena = arena
        self.rank, self.world = arena.rank, arena.world
        self.side: Optional[torch.cuda.Stream] = None   # stream of the copy-engine gather
        self.watchdog = None                            # host-side bound on the gather's stream waits
        self.calls = {"attn": 0, "mlp": 0}              # block halves run on the fused path (tests read this)

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
                save_pre=False, dgelu_aux=None, via_copy_engine: Optional[bool] = None, out=None,
                keep_gathered: bool = False):
        """``concat_ranks(x_shard) @ w^T`` (or ``@ w`` with ``b_mn``) with the usual fused epilogues. No barrier in
        front: every rank publishes its shard with a one-way signal and the GEMM's TMA thread waits (bounded) for
        what it needs right before its first tile of a peer's rows, while the tiles of the own shard are computing.

        Two transports. Direct: the GEMM's TMA loads read the peers' shards over NVLink - every output column tile
        fetches its A tiles again (a peer's memory is not cached in the local L2), so this is for outputs of one
        column tile (N <= 256). Copy engine (default for wider outputs): a side stream waits for each peer's signal
        with a stream memory operation, copies the shard into local memory with the copy engines and publishes
        "ready" with another stream memory operation, all without an SM (a kernel could not be scheduled beside the
        persistent GEMM); the GEMM reads local memory and waits on the ready words. The shard crosses NVLink once.
        The staged shards stay untouched until the next barrier of the group (``gemm_rs`` ends with one).

        ``out``: where the product goes (for example a buffer of another symmetric arena). ``keep_gathered``: use the
        copy-engine transport, let it place the own shard too, and return ``(product, gathered operand)`` - the
        weight-gradient product of the backward pass contracts over the gathered rows and so needs them once."""
        staged = self.stage(x_shard)
        epoch = self.arena.publish()
        N = w.shape[1] if b_mn else w.shape[0]
        if via_copy_engine is None:
            via_copy_engine = N > 256
        if keep_gathered:
            via_copy_engine = True
        kw = dict(b_mn=b_mn, bias=bias, gelu=gelu, save_pre=save_pre, dgelu_aux=dgelu_aux, rank=self.rank, a_epoch=epoch,
                  a_budget_ns=PEER_WAIT_NS, out=out)
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
        self.watch_waits()
        _ext.load().gather_shards_async(self.side.cuda_stream, gathered.data_ptr(), self.arena.peer_ptrs(staged),
                                        self.rank, rows, row_bytes, chunks, chunk_tiles * 128,
                                        self.arena.signal_flags_ptr, self.arena.ready_flags_ptr, epoch, bool(keep_gathered))
        local = [gathered.data_ptr() + r * nbytes for r in range(self.world)]
        local[self.rank] = staged.data_ptr()            # the own shard is read in place
        res = gemm(staged, w, a_peers=local, a_flags=self.arena.ready_flags_ptr, a_interleave=False, a_chunks=chunks, **kw)
        main.wait_stream(self.side)                     # the peers' shards have been read before this rank's next barrier
        if keep_gathered:
            return res, gathered
        return res

    def watch_waits(self) -> None:
        """The copy-engine gather waits for a peer's signal with a stream memory operation, which has no time limit of
        its own. A host watchdog (``terra_b200.runtime.watchdog.StreamWaitWatchdog``) bounds it: if the side stream has
        not drained ``TERRA_PEER_WAIT_MS`` after the last gather was queued, it releases the waits and records the
        failure for the training loop to raise."""
        from ..runtime.watchdog import StreamWaitWatchdog

        if self.watchdog is None:
            self.watchdog = StreamWaitWatchdog(self.arena, lambda: self.side)
        self.watchdog.arm()

    # ---- GEMM -> reduce-scatter
    def gemm_rs(self, a: torch.Tensor, w: torch.Tensor, *, b_mn: bool = False, exact: bool = False, bias=None,
                residual=None) -> torch.Tensor:
        """Row block ``rank`` of ``sum_ranks(a @ w^T)``: ``[M / world, N]``, bf16 (fp32 with ``exact``).

        Default: every rank stores its bf16 partial of row block j into its own slot of owner j's staging (plain
        16-byte stores over NVLink, no zeroing, no atomics); after one barrier the owner adds the slots up in fp32,
        together with ``bias`` (bf16 ``[N]``: the replicated bias of a row-parallel layer) and ``residual`` (bf16, the
        block's shortcut) when given. ``exact``: fp32 vector reductions into the owner's accumulation buffer instead
        (twice the NVLink bytes and a zero + barrier in front, but the partials are not rounded to bf16)."""
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
            if bias is not None:
                acc = acc + bias.float()
            if residual is not None:
                acc = acc + residual.float()
            return acc
        slots = self.arena.alloc((self.world, rows, N), torch.bfloat16)
        gemm(a, w, b_mn=b_mn, out=slots, out_peers=self.arena.peer_ptrs(slots), rank=self.rank)
        self.arena.barrier()            # every rank's partial has landed in this rank's slots
        out = torch.empty(rows, N, dtype=torch.bfloat16, device=a.device)
        _ext.load().sum_slots(slots, out, bias, residual)
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


# ------------------------------------------------------------------------------------------------ whole block halves
def _padded(arena, rows, rows_pad, cols, dtype=torch.bfloat16):
    """``[rows_pad, cols]`` symmetric buffer; the padding rows (ragged tensor-parallel window counts) are zero."""
    t = arena.alloc((rows_pad, cols), dtype)
    if rows_pad > rows:
        t[rows:].zero_()
    return t


class _TpAttnHalfFn(torch.autograd.Function):
    """x + proj(window_attention(qkv(norm1(x)))) on tensor-parallel shards with both collectives inside the GEMMs:

        LayerNorm (own rows, written into symmetric memory)
        -> all-gather -> [q|k|v] GEMM (column-sharded ``[3C/tp, C]`` operand)      ``ag_gemm``
        -> window attention over the window group's windows, this rank's heads
        -> proj GEMM (row-sharded ``[C, C/tp]``) -> reduce-scatter, + proj_bias + x  ``gemm_rs``

    (reference: the all-gather / reduce-scatter pair around the attention of models/attention.py:759-931). Backward is
    the adjoint: all-gather -> GEMM for d(attention output), GEMM -> reduce-scatter for d(norm1 output); the weight
    gradients contract over the gathered rows, which the copy-engine transport of ``ag_gemm`` leaves in local memory.
    ``rows_pad``: rows per rank of the symmetric buffers (the largest rank's; ranks with fewer windows pad with zeros).
    """

    @staticmethod
    def forward(ctx, x, anchor, pk, geo, num_heads, shifted, use_mask, scale, attn_comm, comm: TpFusedComm, rows_pad,
                ragged):
        from .blocks import LN_EPS

        ext = _ext.load()
        rows, C = x.shape
        Cl = pk.qkv_w.shape[0] // 3
        tp = comm.world
        M = rows_pad * tp
        short = rows_pad > rows       # this rank holds fewer windows than the buffers have room for
        xn = _padded(comm.arena, rows, rows_pad, C)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty_like(mean)
        ext.layernorm_fwd(x, pk.ln_w, pk.ln_b, xn[:rows], mean, rstd, LN_EPS)
        save_gathered = tp <= 2
        if attn_comm is not None:
            qkv = attn_comm.alloc_qkv(M, 3 * Cl)
        else:
            qkv = torch.empty(M, 3 * Cl, dtype=torch.bfloat16, device=x.device)
        res = comm.ag_gemm(xn, pk.qkv_w, bias=pk.qkv_b, out=qkv, keep_gathered=save_gathered)
        xn_full = res[1] if save_gathered else None
        if attn_comm is not None:
            o, qkv_ptrs, out_ptrs = attn_comm.attn_forward_buffers(qkv, Cl, shifted)
        else:
            o = torch.empty(M, Cl, dtype=torch.bfloat16, device=x.device)
            qkv_ptrs, out_ptrs = [qkv.data_ptr()], [o.data_ptr()]
        if ragged:
            o.zero_()       # some rank's chunk ends in padding windows, which the attention kernel never visits
        sh, sw = geo.shift(shifted)
        from .attention import launch_window_attn_fwd

        launch_window_attn_fwd(ext, qkv_ptrs, out_ptrs, pk.bias_table, geo, Cl, num_heads, sh, sw, use_mask and shifted,
                               scale, x.device)
        if attn_comm is not None:
            o, qkv = attn_comm.attn_forward_done(o, qkv, shifted)
        if short:
            y = comm.gemm_rs(o, pk.proj_w, bias=pk.proj_b)[:rows] + x
        else:
            y = comm.gemm_rs(o, pk.proj_w, bias=pk.proj_b, residual=x)
        ctx.save_for_backward(x, mean, rstd, xn_full if save_gathered else xn, qkv, o)
        ctx.pk, ctx.geo, ctx.args = pk, geo, (num_heads, shifted, use_mask, scale, rows_pad, save_gathered, ragged)
        ctx.attn_comm, ctx.comm = attn_comm, comm
        return y

    @staticmethod
    def backward(ctx, dy):
        from .blocks import bias_grad_accumulate, layernorm_bwd_cuda, wgrad_accumulate

        ext = _ext.load()
        x, mean, rstd, xn_saved, qkv, o = ctx.saved_tensors
        pk, geo, attn_comm, comm = ctx.pk, ctx.geo, ctx.attn_comm, ctx.comm
        num_heads, shifted, use_mask, scale, rows_pad, save_gathered, ragged = ctx.args
        rows, C = x.shape
        Cl = pk.qkv_w.shape[0] // 3
        M = rows_pad * comm.world
        short = rows_pad > rows
        dy = dy.contiguous()
        bias_grad_accumulate(dy, pk.proj_bg)
        dy_s = _padded(comm.arena, rows, rows_pad, C)
        dy_s[:rows].copy_(dy)
        if attn_comm is not None:
            do = attn_comm.alloc_dout(M, Cl)
        else:
            do = torch.empty(M, Cl, dtype=torch.bfloat16, device=x.device)
        # d(attention output) = gather(dy) @ proj_w: all-gather -> GEMM (the adjoint of the reduce-scatter)
        _, dy_full = comm.ag_gemm(dy_s, pk.proj_w, b_mn=True, out=do, keep_gathered=True)
        wgrad_accumulate(dy_full, o, pk.proj_wg)
        if attn_comm is not None:
            dqkv, qkv_ptrs, dout_ptrs, dqkv_ptrs = attn_comm.attn_backward_buffers(qkv, do, shifted)
        else:
            dqkv = torch.empty_like(qkv)
            qkv_ptrs, dout_ptrs, dqkv_ptrs = [qkv.data_ptr()], [do.data_ptr()], [dqkv.data_ptr()]
        if ragged:
            dqkv.zero_()
        sh, sw = geo.shift(shifted)
        from .attention import launch_window_attn_bwd

        launch_window_attn_bwd(ext, qkv_ptrs, dout_ptrs, dqkv_ptrs, pk.bias_table, pk.bias_table_g, geo, Cl, num_heads, sh,
                               sw, use_mask and shifted, scale, x.device)
        if attn_comm is not None:
            dqkv = attn_comm.attn_backward_done(dqkv, shifted)
        if save_gathered:
            xn_full = xn_saved
        else:
            xn_s = comm.stage(xn_saved)
            comm.arena.barrier()
            xn_full = _gather_rows(comm, xn_s)
        wgrad_accumulate(dqkv, xn_full, pk.qkv_wg, pk.qkv_bg)
        # d(norm1 output) = reduce-scatter(dqkv @ qkv_w): GEMM -> reduce-scatter (the adjoint of the all-gather)
        dxn = comm.gemm_rs(dqkv, pk.qkv_w, b_mn=True)
        dx = layernorm_bwd_cuda(dxn[:rows] if short else dxn, x, pk.ln_w, mean, rstd, pk.ln_wg, pk.ln_bg, dres=dy)
        return (dx,) + (None,) * 11


class _TpMlpHalfFn(torch.autograd.Function):
    """x + fc2(gelu(fc1(norm2(x)))) + bias2 on tensor-parallel shards: LayerNorm into symmetric memory, all-gather ->
    fc1 GEMM (+bias, GELU, pre-activation kept), fc2 GEMM -> reduce-scatter (+bias2 +x in the owner's sum)
    (reference: models/mlp.py:478-530)."""

    @staticmethod
    def forward(ctx, x, anchor, pk, comm: TpFusedComm, rows_pad):
        from .blocks import LN_EPS

        ext = _ext.load()
        rows, C = x.shape
        short = rows_pad > rows
        xn = _padded(comm.arena, rows, rows_pad, C)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty_like(mean)
        ext.layernorm_fwd(x, pk.ln_w, pk.ln_b, xn[:rows], mean, rstd, LN_EPS)
        save_gathered = comm.world <= 2
        res = comm.ag_gemm(xn, pk.fc1_w, bias=pk.fc1_b, gelu=True, save_pre=True, keep_gathered=save_gathered)
        (act, pre), xn_full = (res if save_gathered else (res, None))
        if short:
            y = comm.gemm_rs(act, pk.fc2_w, bias=pk.bias2)[:rows] + x
        else:
            y = comm.gemm_rs(act, pk.fc2_w, bias=pk.bias2, residual=x)
        ctx.save_for_backward(x, mean, rstd, xn_full if save_gathered else xn, pre, act)
        ctx.pk, ctx.comm, ctx.args = pk, comm, (rows_pad, save_gathered)
        return y

    @staticmethod
    def backward(ctx, dy):
        from .blocks import bias_grad_accumulate, layernorm_bwd_cuda, wgrad_accumulate

        x, mean, rstd, xn_saved, pre, act = ctx.saved_tensors
        pk, comm = ctx.pk, ctx.comm
        rows_pad, save_gathered = ctx.args
        rows, C = x.shape
        short = rows_pad > rows
        dy = dy.contiguous()
        bias_grad_accumulate(dy, pk.bias2_g)
        dy_s = _padded(comm.arena, rows, rows_pad, C)
        dy_s[:rows].copy_(dy)
        dpre, dy_full = comm.ag_gemm(dy_s, pk.fc2_w, b_mn=True, dgelu_aux=pre, keep_gathered=True)
        wgrad_accumulate(dy_full, act, pk.fc2_wg)
        if save_gathered:
            xn_full = xn_saved
        else:
            xn_s = comm.stage(xn_saved)
            comm.arena.barrier()
            xn_full = _gather_rows(comm, xn_s)
        wgrad_accumulate(dpre, xn_full, pk.fc1_wg, pk.fc1_bg)
        dxn = comm.gemm_rs(dpre, pk.fc1_w, b_mn=True)
        dx = layernorm_bwd_cuda(dxn[:rows] if short else dxn, x, pk.ln_w, mean, rstd, pk.ln_wg, pk.ln_bg, dres=dy)
        return dx, None, None, None, None


def tp_attention_half(x, mod, geo, attn_comm, comm: TpFusedComm, rows_pad: int, ragged: bool = False):
    """The attention half of a Swin block on tensor-parallel shards (``mod``: a ``SwinAttentionHalf`` of the
    factorised build: q/k/v column-sharded, proj row-sharded, replicated ``proj_bias``). ``ragged``: the window
    count of the group is not a multiple of the tensor-parallel size, so some rank's chunk of the gathered buffers
    ends in padding windows (a property of the group: every rank passes the same value)."""
    from .blocks import ParamPack

    comm.calls["attn"] += 1
    a = mod.attn
    fused = a.fused
    has_bias = a.use_relative_position_bias
    pk = ParamPack(
        ln_w=mod.norm1.weight.bf16, ln_b=mod.norm1.bias.bf16, ln_wg=mod.norm1.weight.grad, ln_bg=mod.norm1.bias.grad,
        qkv_w=fused["qkv_weight"].bf16, qkv_b=fused["qkv_bias"].bf16, qkv_wg=fused["qkv_weight"].grad,
        qkv_bg=fused["qkv_bias"].grad, proj_w=a.proj.weight.bf16, proj_wg=a.proj.weight.grad,
        proj_b=a.proj_bias.bf16, proj_bg=a.proj_bias.grad,
        bias_table=fp32_values(a.relative_position_bias_table) if has_bias else None,
        bias_table_g=a.relative_position_bias_table.grad if has_bias else None)
    return _TpAttnHalfFn.apply(x, mod.norm1.weight, pk, geo, a.num_heads, mod.shifted, mod.use_attn_mask, a.scale,
                               attn_comm, comm, rows_pad, ragged)


def tp_mlp_half(x, mod, comm: TpFusedComm, rows_pad: int):
    """The MLP half of a Swin block on tensor-parallel shards (``linear1`` column-sharded, ``linear2`` row-sharded,
    replicated ``bias2``)."""
    from .blocks import ParamPack

    comm.calls["mlp"] += 1
    l1, l2 = mod.linear1, mod.linear2
    pk = ParamPack(
        ln_w=mod.norm2.weight.bf16, ln_b=mod.norm2.bias.bf16, ln_wg=mod.norm2.weight.grad, ln_bg=mod.norm2.bias.grad,
        fc1_w=l1.weight.bf16, fc1_b=l1.bias.bf16, fc1_wg=l1.weight.grad, fc1_bg=l1.bias.grad,
        fc2_w=l2.weight.bf16, fc2_wg=l2.weight.grad, bias2=mod.bias2.bf16, bias2_g=mod.bias2.grad)
    return _TpMlpHalfFn.apply(x, mod.norm2.weight, pk, comm, rows_pad)
