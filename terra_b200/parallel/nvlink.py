"""NVLink / NVSwitch backend: symmetric (peer-mapped) arenas and the operators that use them.

Every rank of a group allocates the same arena layout through ``torch.distributed._symmetric_memory`` (PyTorch does
the handle exchange and the peer mapping); kernels then address a peer's copy of a buffer as
``peer_base + same offset``. On top of that:

* ``FusedAttnComm``  - window attention whose CTAs read q/k/v rows of halo windows (window parallel) and of the other
  token shards (sequence parallel) straight from the owners' buffers and store outputs to the tokens' home rows;
  the only collectives left are two flag barriers around the shifted / sharded blocks;
* ``FusedDistAdamW`` - the sharded optimizer step as one kernel: P2P reduce of the owned gradient range, fp32
  AdamW, P2P store of the bf16 working copy to every replica;
* small helpers: barrier on a symmetric signal pad (monotonic epochs, bounded spin, status word on expiry), sum of
  small per-rank vectors (GroupNorm statistics).

No TMA load here fans out over a cluster; remote data is read with plain loads or per-CTA TMA.
"""
from __future__ import annotations

import os

from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from .. import _ext
from ..ops.gemm import status_word

COMM_MAX_PEERS = 16
PAD_BYTES = 4096            # signal pads at the start of every arena
# time budget of a device-side wait on a peer (nanoseconds of the GPU's global timer); TERRA_PEER_WAIT_MS overrides
BARRIER_SPIN_LIMIT = int(float(os.environ.get("TERRA_PEER_WAIT_MS", "5000")) * 1e6)
# debugging aid: wipe the per-step region of every symmetric arena with NaN patterns at each reset (see reset())
ARENA_POISON = os.environ.get("TERRA_ARENA_POISON", "0") == "1"


def _symm():
    import torch.distributed._symmetric_memory as symm_mem

    return symm_mem


class _RawBytes:
    """CUDA-array-interface view of ``nbytes`` at ``ptr``; keeps ``owner`` alive."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.owner = owner
        self.__cuda_array_interface__ = {"shape": (int(nbytes),), "typestr": "|u1", "data": (int(ptr), False), "version": 2}


_GROUP_OF_NAME = {}      # group name -> the process-group object that was registered for symmetric memory under it


def _register_group(symm_mem, group) -> None:
    """Register ``group`` with torch's symmetric-memory layer. That layer keeps a process-wide table keyed by the group's
    NAME and never re-registers a name it knows; names are handed out from a counter that ``destroy_process_group``
    resets. So after a process has torn its groups down and built another topology, a new group inherits the name - and
    with it the rank, size and store - of a group of the old topology, and the rendezvous waits on a dead store for the
    wrong number of peers. A name that is known for a different group object is therefore dropped before registering."""
    name = group.group_name
    table = getattr(symm_mem, "_group_name_to_store", None)
    if _GROUP_OF_NAME.get(name) is not group and isinstance(table, dict):
        table.pop(name, None)
    _GROUP_OF_NAME[name] = group
    try:
        symm_mem.enable_symm_mem_for_group(name)
    except Exception:
        pass


class SymmetricArena:
    """Bump allocator over one symmetric allocation shared (by layout) with the ranks of ``group``."""

    def __init__(self, group, nbytes: int, device: torch.device):
        symm_mem = _symm()
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.nbytes = int(nbytes + PAD_BYTES + 255) // 256 * 256
        _register_group(symm_mem, group)
        self.buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.hdl = symm_mem.rendezvous(self.buf, group=group)
        self.base_ptrs: List[int] = [int(p) for p in self.hdl.buffer_ptrs]
        if self.base_ptrs[self.rank] != self.buf.data_ptr():
            # some versions report the local mapping under a different address; use the tensor's
            self.base_ptrs[self.rank] = self.buf.data_ptr()
        self.cursor = PAD_BYTES
        self.persistent_end = PAD_BYTES
        self.epoch = 0
        torch.cuda.synchronize(device)
        dist.barrier(group)

    # ---- allocation
    def alloc(self, shape, dtype, persistent: bool = False) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        start = (self.cursor + 255) // 256 * 256
        if start + nbytes > self.nbytes:
            raise RuntimeError(f"symmetric arena exhausted: need {start + nbytes} of {self.nbytes} bytes "
                               "(raise TERRA_SYMM_ARENA_GB)")
        self.cursor = start + nbytes
        if persistent:
            if start != (self.persistent_end + 255) // 256 * 256:
                raise RuntimeError("persistent symmetric allocations must come before any per-step allocation")
            self.persistent_end = self.cursor
        # A fresh alias of the bytes (own autograd version counter): tensors carved from one arena must not look
        # like views of each other, or an in-place update of one (gradient accumulation) would invalidate another
        # that autograd saved (the bf16 working copy).
        raw = torch.as_tensor(_RawBytes(self.buf.data_ptr() + start, nbytes, self.buf), device=self.buf.device)
        return raw.view(dtype).view(*shape)

    def reset(self) -> None:
        """Forget the per-step allocations (call between steps, when no kernel of the previous step is pending
        on a peer: the last cross-rank access of a step is followed by a barrier).

        ``TERRA_ARENA_POISON=1`` (race hunting): the region the step used is filled with 0xFF bytes first - NaN as
        bf16 and as fp32 - so that a kernel which reads a peer buffer before its producer wrote it, or a buffer of
        the previous step, turns the loss into NaN instead of silently using stale numbers. A barrier follows the
        fill: a faster peer must not push the new step's rows into this region before it has been wiped."""
        if ARENA_POISON and self.cursor > self.persistent_end:
            self.buf[self.persistent_end:self.cursor].fill_(0xFF)
            self.barrier()
        self.cursor = self.persistent_end

    def offset_of(self, t: torch.Tensor) -> int:
        off = t.data_ptr() - self.buf.data_ptr()
        if off < 0 or off >= self.nbytes:
            raise ValueError("tensor is not inside this symmetric arena")
        return off

    def peer_ptrs(self, t: torch.Tensor) -> List[int]:
        off = self.offset_of(t)
        return [b + off for b in self.base_ptrs]

    # ---- synchronisation
    SIGNAL_SLOT = 64       # words [64, 64 + world) of the pad count the one-way "published" signals per source rank

    def publish(self) -> int:
        """One-way signal "everything this rank wrote so far (stream order) is visible"; returns the epoch that the
        consumers wait for. All ranks call it in the same order, so the epochs agree."""
        self.signal_epoch = getattr(self, "signal_epoch", 0) + 1
        _ext.load().peer_signal(self.base_ptrs, self.rank, self.SIGNAL_SLOT)
        return self.signal_epoch

    READY_SLOT = 128       # words [128, 128 + world): "peer's shard has been copied into local memory" (copy-engine gather)

    @property
    def ready_flags_ptr(self) -> int:
        return self.base_ptrs[self.rank] + 4 * self.READY_SLOT

    @property
    def signal_flags_ptr(self) -> int:
        """Device address of this rank's ``[world]`` array of published counts (one per source rank)."""
        return self.base_ptrs[self.rank] + 4 * self.SIGNAL_SLOT

    def release_waits(self) -> None:
        """Satisfy every stream memory-operation wait that may still be queued on this rank's signal words (the
        copy-engine gather waits for a peer's signal without a time limit of its own). Called at shutdown, by the
        host watchdog when such a wait outlives its budget and after a peer was reported lost, so that a dead peer
        cannot keep this process's streams - and its exit - blocked. The words are written with stream memory
        operations (no SM needed, so a resident persistent kernel cannot delay them). The arena is unusable for
        signalling afterwards."""
        ext = _ext.load()
        side = torch.cuda.Stream(self.buf.device)
        base = self.base_ptrs[self.rank] + 4 * self.SIGNAL_SLOT
        for i in range(COMM_MAX_PEERS):
            ext.stream_write_value(side.cuda_stream, base + 4 * i, 0x7F7F7F7F)     # above any epoch a run reaches
        side.synchronize()
        self.released = True

    def barrier(self) -> None:
        """Stream-ordered barrier over the group (device side; the host does not wait)."""
        self.epoch += 1
        _ext.load().peer_barrier(self.base_ptrs, self.rank, self.epoch, status_word(self.buf.device), BARRIER_SPIN_LIMIT)


class FusedAttnComm:
    """Peer access for ``window_attn`` over the (window group x token shard) ranks that share a TP rank."""

    fused = True

    def __init__(self, arena: SymmetricArena, n_wg: int, sp: int):
        self.arena = arena
        self.world = arena.world
        self.n_wg, self.sp = n_wg, sp
        if arena.world != n_wg * sp:
            raise ValueError(f"attention peer group has {arena.world} ranks, expected {n_wg} x {sp}")
        self.max_rows: Optional[int] = None

    def _needs_peers(self, shifted: bool) -> bool:
        return self.sp > 1 or (shifted and self.n_wg > 1)

    def _rows(self, rows: int) -> int:
        # every rank must advance the arena identically: size by the largest shard (ragged ownership)
        if self.max_rows is None:
            t = torch.tensor([rows], device=self.arena.buf.device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.arena.group)
            self.max_rows = int(t.item())
        return max(rows, self.max_rows)

    def alloc_qkv(self, rows, cols):
        full = self.arena.alloc((self._rows(rows), cols), torch.bfloat16)
        return full[:rows]

    def attn_forward_buffers(self, qkv, C, shifted):
        rows = qkv.shape[0]
        o = self.arena.alloc((self._rows(rows), C), torch.bfloat16)[:rows]
        if self._needs_peers(shifted):
            self.arena.barrier()                       # every peer's q/k/v is complete
        return o, self.arena.peer_ptrs(qkv), self.arena.peer_ptrs(o)

    def attn_forward_done(self, o, qkv, shifted):
        if self._needs_peers(shifted):
            self.arena.barrier()                       # every peer's stores into my rows have landed
        return o, qkv

    def alloc_dout(self, rows, C):
        return self.arena.alloc((self._rows(rows), C), torch.bfloat16)[:rows]

    def alloc_f32(self, rows, cols):
        """Per-row fp32 side data that peers read or write (log-sum-exp, row dots of large-window attention)."""
        return self.arena.alloc((self._rows(rows), cols), torch.float32)[:rows]

    def attn_backward_buffers(self, qkv, do, shifted):
        rows = qkv.shape[0]
        dqkv = self.arena.alloc((self._rows(rows), qkv.shape[1]), torch.bfloat16)[:rows]
        if self._needs_peers(shifted):
            self.arena.barrier()
        return dqkv, self.arena.peer_ptrs(qkv), self.arena.peer_ptrs(do), self.arena.peer_ptrs(dqkv)

    def attn_backward_done(self, dqkv, shifted):
        if self._needs_peers(shifted):
            self.arena.barrier()
        return dqkv


class PeerDomain:
    """Row-stripe (domain-parallel) communication of the sampling blocks over peer memory: the halo rows of the
    3 x 3 convolutions are pushed into the neighbours' receive buffers by one kernel (``halo_push``), and the small
    all-reduces of the distributed GroupNorm (statistics forward, two sums backward) are one single-block kernel
    (``peer_allreduce_small``). No NCCL call is left in the convolution stage (reference:
    credit/domain_parallel/halo_exchange.py:18-157, layers.py:18-84)."""

    FROM_PREV, FROM_NEXT, TICKET, SMALL_FLAGS = 256, 257, 258, 272      # words of the arena's signal pad
    SMALL_CAPACITY = 8192

    def __init__(self, arena: SymmetricArena):
        self.arena = arena
        self.rank, self.world = arena.rank, arena.world
        self.slots = arena.alloc((2, self.world, self.SMALL_CAPACITY), torch.float32, persistent=True)
        self.halo_epoch = 0
        self.small_epoch = 0

    def _word(self, rank: int, index: int) -> int:
        return self.arena.base_ptrs[rank] + 4 * index

    def exchange_rows(self, top: torch.Tensor, bot: torch.Tensor):
        """Send ``top`` (this stripe's first row) to the previous rank and ``bot`` (its last row) to the next one;
        returns ``(row above, row below)`` as tensors in this rank's symmetric memory (``None`` at the grid edges).
        Every rank of the group calls this the same number of times per step."""
        ext = _ext.load()
        top, bot = top.contiguous(), bot.contiguous()
        lo = self.arena.alloc(tuple(top.shape), top.dtype)       # receives the previous rank's last row
        hi = self.arena.alloc(tuple(bot.shape), bot.dtype)       # receives the next rank's first row
        self.halo_epoch += 1
        has_prev, has_next = self.rank > 0, self.rank < self.world - 1
        nbytes = top.numel() * top.element_size()
        ext.halo_push(
            top.data_ptr(), bot.data_ptr(),
            self.arena.peer_ptrs(hi)[self.rank - 1] if has_prev else 0,      # my first row is the previous rank's row below
            self.arena.peer_ptrs(lo)[self.rank + 1] if has_next else 0,
            nbytes,
            self._word(self.rank - 1, self.FROM_NEXT) if has_prev else 0,
            self._word(self.rank + 1, self.FROM_PREV) if has_next else 0,
            self._word(self.rank, self.FROM_PREV) if has_prev else 0,
            self._word(self.rank, self.FROM_NEXT) if has_next else 0,
            self.halo_epoch, self._word(self.rank, self.TICKET), status_word(self.arena.buf.device), BARRIER_SPIN_LIMIT)
        return (lo if has_prev else None), (hi if has_next else None)

    def gather_rows(self, x: torch.Tensor, src_rank: torch.Tensor, src_row: torch.Tensor) -> torch.Tensor:
        """``out[i] = row src_row[i] of rank src_rank[i]'s x`` (int32 device tables; every rank passes its own ``x``,
        all with the same number of columns). The general stripe <-> window relayout: an all-to-all-v in which the
        receiver pulls exactly the rows it owns, in one kernel, instead of an all-gather of the whole activation."""
        ext = _ext.load()
        rows = torch.tensor([x.shape[0]], device=x.device)
        if not hasattr(self, "_max_rows"):
            self._max_rows = {}
        key = (x.shape[0], x.shape[1])
        if key not in self._max_rows:
            dist.all_reduce(rows, op=dist.ReduceOp.MAX, group=self.arena.group)      # symmetric allocation: largest shard
            self._max_rows[key] = int(rows.item())
        staged = self.arena.alloc((self._max_rows[key], x.shape[1]), x.dtype)[:x.shape[0]]
        staged.copy_(x)
        self.arena.barrier()                      # every rank's rows are staged
        out = torch.empty(src_rank.numel(), x.shape[1], dtype=x.dtype, device=x.device)
        ext.peer_gather_indexed(out, self.arena.peer_ptrs(staged), src_rank, src_row, self._max_rows[key],
                                status_word(x.device))
        return out

    def all_reduce_small(self, t: torch.Tensor) -> torch.Tensor:
        """Sum of a small fp32 tensor over the group (a new tensor)."""
        ext = _ext.load()
        flat = t.contiguous().view(-1)
        if flat.numel() > self.SMALL_CAPACITY:
            raise ValueError(f"peer all-reduce holds at most {self.SMALL_CAPACITY} values, got {flat.numel()}")
        out = torch.empty_like(flat)
        self.small_epoch += 1
        ext.peer_allreduce_small(self.arena.peer_ptrs(self.slots),
                                 [self._word(r, self.SMALL_FLAGS) for r in range(self.world)], flat, out, self.rank,
                                 self.SMALL_CAPACITY, self.small_epoch, status_word(self.arena.buf.device),
                                 BARRIER_SPIN_LIMIT)
        return out.view(t.shape)


class FusedDistAdamW:
    """One kernel per parameter class: reduce-scatter + AdamW + all-gather over peer memory."""

    def __init__(self, arenas: Dict[str, SymmetricArena], grad_views: Dict[str, torch.Tensor],
                 bf16_views: Dict[str, torch.Tensor]):
        self.arenas, self.grad_views, self.bf16_views = arenas, grad_views, bf16_views

    def step(self, opt, g0, scale):
        ext = _ext.load()
        a = opt.arena
        b1, b2 = g0["betas"]
        for sh in opt.shards:
            ar = self.arenas.get(sh.label)
            if ar is None or sh.size == 1:
                opt.portable_shard_step(sh, g0, scale)
                continue
            n_own = sh.hi - sh.lo
            if sh.exp_avg is None:
                sh.exp_avg = torch.zeros(max(n_own, 1), dtype=torch.float32, device=a.master.device)
                sh.exp_avg_sq = torch.zeros_like(sh.exp_avg)
            ar.barrier()                                   # every replica's gradients are final
            ext.dist_adamw_step(ar.peer_ptrs(self.grad_views[sh.label]), ar.peer_ptrs(self.bf16_views[sh.label]),
                                a.master, sh.exp_avg, sh.exp_avg_sq, sh.lo, n_own, g0["lr"], b1, b2, g0["eps"],
                                g0["weight_decay"], opt.step_count, scale)
            ar.barrier()                                   # every replica's working copy is complete
            opt._masters_stale = True


def attach(model, optimizer, manager) -> None:
    """Switch a freshly built (model, optimizer) pair to the peer-memory paths."""
    import os

    from ..optim.distributed_adamw import DistributedAdamW
    from ..utils.flat_params import ParamArena, get_arena

    device = next(model.parameters()).device
    pctx = model.pctx
    gb = float(os.environ.get("TERRA_SYMM_ARENA_GB", "0"))
    # ---- attention peers: (window group x token shard) at this TP rank
    if pctx.n_wg * pctx.sp > 1 and pctx.contiguous:
        if gb <= 0:
            rows = max(len(w) for w in pctx.windows_of) * pctx.shardN * pctx.B
            C = model.embedding_dim // pctx.tp
            per_layer = rows * C * 2 * (3 + 1 + 1 + 3) + rows * 64 * 4 * 2   # qkv, o, do, dqkv; lse / row dots (large windows)
            nbytes = int(per_layer * model.num_layers * 1.25) + (64 << 20)
        else:
            nbytes = int(gb * (1 << 30))
        arena = SymmetricArena(manager.xfmr_tp_param_group, nbytes, device)
        pctx.fused_comm = FusedAttnComm(arena, pctx.n_wg, pctx.sp)
        pctx.attn_arena = arena
    # ---- sampling blocks: halo rows and GroupNorm sums over peer memory
    if manager.wp_size > 1 and getattr(model, "has_sampling", False) and os.environ.get("TERRA_PEER_HALO", "1") != "0":
        a = model
        w_tok = a.patches_resolution[1]
        row = pctx.B * w_tok * model.embedding_dim * 4          # one fp32 boundary row at patch resolution
        nbytes = 48 * row + 2 * COMM_MAX_PEERS * PeerDomain.SMALL_CAPACITY * 4 + (16 << 20)
        if not pctx.local_relayout:
            # general relayout: the activation shard is staged twice forward, twice backward (and once more each when
            # the surrounding segment is recomputed)
            shard = pctx.B * (pctx.Ht // pctx.world + 1) * pctx.Wt * model.embedding_dim * 2
            win = pctx.B * (max(len(w) for w in pctx.windows_of) // pctx.tp + 1) * pctx.N * model.embedding_dim * 2
            nbytes += 4 * (shard + win) + (16 << 20)
        pctx.dom_arena = SymmetricArena(manager.window_parallel_group, nbytes, device)
        pctx.dom.peer = PeerDomain(pctx.dom_arena)
    # ---- tensor-parallel MLP: fc1 / fc2 with the all-gather / reduce-scatter fused into the GEMMs
    if pctx.tp > 1 and os.environ.get("TERRA_TP_FUSED", "1") != "0":
        from ..ops.tp_fused import TpFusedComm

        rows = max(pctx.tp_sizes_windows) * pctx.shardN * pctx.B
        C, F = model.embedding_dim, 4 * model.embedding_dim
        # per block half, forward + backward: staged xn, dy (bf16), reduce-scatter slots (bf16 x tp x 2); two halves per
        # layer; recomputed segments stage their forward buffers a second time within the step
        per_layer = 2 * rows * (2 * C * 2 + 2 * pctx.tp * C * 2)
        nbytes = int(per_layer * model.num_layers * 1.5) + (64 << 20)
        pctx.tp_arena = SymmetricArena(manager.xfmr_tp_group, nbytes, device)
        pctx.tp_comm = TpFusedComm(pctx.tp_arena)
    # ---- sharded optimizer: gradients and working copy must be peer visible. One symmetric allocation is mapped
    # for one group, so the largest parameter class gets the fused kernel; other classes (TP shards, whose replica
    # group differs) keep the collective path on the same buffers.
    if isinstance(optimizer, DistributedAdamW):
        pa = get_arena(model)
        cands = [sh for sh in optimizer.shards if sh.size > 1]
        if cands:
            sh = max(cands, key=lambda s: s.end - s.start)
            n = pa.numel
            ar = SymmetricArena(sh.group, n * 4 + n * 2 + 8192, device)
            g = ar.alloc((n,), torch.float32, persistent=True)
            b = ar.alloc((n,), torch.bfloat16, persistent=True)
            pa.rebind(g, b)
            optimizer.fused = FusedDistAdamW({sh.label: ar}, {sh.label: g}, {sh.label: b})


def reset_step_arenas(model) -> None:
    for name in ("attn_arena", "tp_arena", "dom_arena"):
        arena = getattr(model.pctx, name, None)
        if arena is not None:
            arena.reset()
