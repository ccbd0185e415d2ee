"""Parameter sharding: every rank keeps 1 / n of each unit's parameters and gathers a unit only while it runs.

This is the role the reference gives to FSDP under ``optimizer_config`` 5, 7, 8 and 9 and to DeepSpeed ZeRO stage 3
(models/model_utils/get_model.py:144-171 block wrapping, :280-344 the TP-aware variant, :1196-1283 the configurations).
The design here follows the flat arenas instead of wrapping modules:

* A *unit* is a group of consecutive transformer blocks (``blocks_per_unit``, the reference's ``FSDP_WRAPPER_CFG``); every
  other parameter (patch embedding / recovery, sampling blocks) belongs to the *root* unit, as in the reference's default
  ``FSDP_SAMPLING_WRAPPER_CFG: 0``. With ``sampling_units`` (that key at 1 or 2) the patch embedding, the down block, the
  up block and the patch recovery are units of their own; the model runs those pieces as functions, so it brackets them
  with ``run_in_unit`` instead of module hooks. ``whole_model`` (config 5) makes the root the only unit.
* Each unit owns a flat arena (``ParamArena`` over its parameters): fp32 values, fp32 gradients and, on the GPU, the bf16
  working copy that the kernels read. The arena is cut per communication label exactly as the sharded optimizer cuts the
  model-wide arena, so TP-sharded parameters are split over the ranks that replicate them (fixed TP rank) and everything
  else over the full replica group: that is the reference's configuration 9; 7 and 8 are the same code with one label.
* Between uses only the owned slices exist (``own_master``, ``own_work``, ``own_grad`` and the optimizer's moments). The
  flat buffers keep their tensor objects, with the storage shrunk to nothing, so every view (``p.data``, ``p.bf16``,
  ``p.grad``, the fused q/k/v views) stays valid and sees the gathered values once the storage is back.
* Hooks drive the schedule: a unit is all-gathered before its first block runs and released after its last block; the
  output of each block carries a gradient hook that gathers the unit again and brings its gradient buffer back before
  the backward pass enters it. A unit's gradients are reduce-scattered to their owners, and the unit released, when the
  backward pass enters the next unit (units are left in reverse forward order), the rest in ``finish_backward``. A forward
  pass that runs inside the backward pass (activation recompute) leaves its units resident for the gradient computation
  that follows. The root unit stays resident from the start of the forward pass to ``finish_backward``.
* ``prefetch: overlap`` starts the all-gather of the neighbouring unit (next in forward, previous in backward)
  asynchronously before the current unit computes, and starts a unit's reduce-scatter when the backward pass leaves
  it without waiting for it (it is folded in when the next unit is left, or in ``finish_backward``); the collectives
  run on the backend's own stream / thread.

Not run on a GPU so far: the CPU (gloo) ranks exercise the schedule, the collectives and the optimizer math.
"""
from __future__ import annotations

import contextlib
import math
from typing import Callable, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..utils.flat_params import ALIGN, ParamArena

PREFETCH_POLICIES = ("none", "overlap", "conservative")


def _free(t: Optional[torch.Tensor]) -> None:
    if t is not None and t.untyped_storage().size() != 0:
        t.untyped_storage().resize_(0)


def _materialise(t: torch.Tensor) -> bool:
    """Give the flat buffer its storage back; ``True`` when it had none."""
    want = t.numel() * t.element_size()
    if t.untyped_storage().size() == want:
        return False
    t.untyped_storage().resize_(want)
    return True


def _inside_backward() -> bool:
    return torch._C._current_graph_task_id() != -1


class OwnedRange:
    """One communication label's segment of a unit's arena and this rank's slice of it."""

    def __init__(self, label, group, rank, size, start, end):
        self.label, self.group, self.rank, self.size = label, group, rank, size
        self.start, self.end = start, end
        if (end - start) % (size * ALIGN):
            raise ValueError(f"segment of {end - start} elements does not split over {size} ranks")
        self.per = (end - start) // size
        self.lo = start + rank * self.per
        self.hi = self.lo + self.per
        self.own_master: Optional[torch.Tensor] = None     # fp32 values of [lo, hi)
        self.own_work: Optional[torch.Tensor] = None       # bf16 copy of them (GPU), the all-gather's source
        self.own_grad: Optional[torch.Tensor] = None       # fp32, summed over the group, accumulated over backward passes
        self.exp_avg: Optional[torch.Tensor] = None
        self.exp_avg_sq: Optional[torch.Tensor] = None


class ShardedUnit:
    def __init__(self, name: str, model, named_params, modules, resolve_group: Callable, index: int,
                 bf16_shadow: Optional[bool] = None):
        self.name, self.index = name, index
        groups = {}
        for _, p in named_params:
            label = getattr(p, "terra_grad_reduce_group", None) or "full"
            if label not in groups:
                groups[label] = resolve_group(label)
        lcm = 16
        for _, _, size in groups.values():
            lcm = lcm * size // math.gcd(lcm, size)
        self.arena = ParamArena(model, bf16_shadow=bf16_shadow, params=named_params, modules=modules,
                                segment_align=ALIGN * lcm)
        self.params = list(self.arena.params)
        if self.arena.bf16 is not None:
            for p in self.params:
                p.terra_master_sharded = True      # fp32 reads go through the widened working copy (ops/packed.py)
        self.ranges: List[OwnedRange] = []
        for seg in self.arena.segments:
            group, rank, size = groups[seg.label]
            r = OwnedRange(seg.label, group, rank, size, seg.start, seg.end)
            r.own_master = self.arena.master[r.lo:r.hi].clone()
            r.own_work = self.arena.bf16[r.lo:r.hi].clone() if self.arena.bf16 is not None else None
            r.own_grad = torch.zeros_like(r.own_master)
            self.ranges.append(r)
        self.resident = True          # the working copy holds gathered values
        self.grad_live = True         # the full gradient buffer has storage and the parameters' .grad point into it
        self.in_backward = False
        self._pending: list = []
        self._reducing: list = []     # (handle, range, received slice) of reduce-scatters in flight
        self.gradient_observer = None  # callable(unit) run before the unit's gradients are reduced (debug reports)
        self.gathers = 0              # counters for tests and reports
        self.reductions = 0
        self.release()
        self.release_grad()
        _free(self.arena.master)      # on the GPU the fp32 values are only materialised for state_dict / load

    # ------------------------------------------------------------------ working copy
    @property
    def work(self) -> torch.Tensor:
        return self.arena.bf16 if self.arena.bf16 is not None else self.arena.master

    def _source(self, r: OwnedRange) -> torch.Tensor:
        return r.own_work if self.arena.bf16 is not None else r.own_master

    def gather(self, async_op: bool = False) -> None:
        if self.resident:
            if not async_op:
                self.wait()
            return
        work = self.work
        _materialise(work)
        with torch.no_grad():
            for r in self.ranges:
                if r.size > 1:
                    self._pending.append(dist.all_gather_into_tensor(work[r.start:r.end], self._source(r), group=r.group,
                                                                     async_op=True))
                else:
                    work[r.start:r.end].copy_(self._source(r))
        self.resident = True
        self.gathers += 1
        if not async_op:
            self.wait()

    def wait(self) -> None:
        for h in self._pending:
            h.wait()
        self._pending = []

    def release(self) -> None:
        self.wait()
        if not self.resident:
            return
        _free(self.work)
        self.resident = False
        if self.arena.bf16 is not None:
            from ..ops.conv import invalidate_packed_weights

            invalidate_packed_weights()          # operands packed from the working copy go with it

    # ------------------------------------------------------------------ gradients
    def materialise_grad(self) -> None:
        self.finish_reduce()              # an earlier pass's reduction still reads the buffer
        if self.grad_live:
            return
        g = self.arena.grad
        _materialise(g)
        g.zero_()
        for p, off in zip(self.arena.params, self.arena.offsets):
            stray = p.grad
            p.grad = g[off:off + p.numel()].view(p.shape)
            if stray is not None:
                p.grad.add_(stray)
        self.grad_live = True

    def release_grad(self) -> None:
        for p in self.arena.params:
            p.grad = None
        _free(self.arena.grad)
        self.grad_live = False

    def has_stray_gradients(self) -> bool:
        return (not self.grad_live) and any(p.grad is not None for p in self.arena.params)

    def reduce_grad(self, async_op: bool = False) -> None:
        """Sum the unit's gradients over each label's replica group, keep the owned slice, drop the rest. With
        ``async_op`` the reduce-scatters are only started (they run on the backend's stream / thread while the backward
        pass goes on); ``finish_reduce`` folds the results in and frees the gradient buffer."""
        if self._reducing:
            if not async_op:
                self.finish_reduce()
            return
        if not self.grad_live:
            return
        if self.gradient_observer is not None:
            self.gradient_observer(self)          # whole-parameter gradients exist until the reduction below
        g = self.arena.grad
        with torch.no_grad():
            for r in self.ranges:
                if r.size > 1:
                    part = torch.empty_like(r.own_grad)
                    h = dist.reduce_scatter_tensor(part, g[r.start:r.end], group=r.group, async_op=True)
                    self._reducing.append((h, r, part))
                else:
                    r.own_grad.add_(g[r.lo:r.hi])
        self.reductions += 1
        if not async_op or not self._reducing:
            self.finish_reduce(force=True)

    def finish_reduce(self, force: bool = False) -> None:
        if not self._reducing and not force:
            return
        with torch.no_grad():
            for h, r, part in self._reducing:
                h.wait()
                r.own_grad.add_(part)
        self._reducing = []
        self.release_grad()

    # ------------------------------------------------------------------ fp32 values (state_dict, load)
    def gather_masters(self) -> None:
        m = self.arena.master
        if self.arena.bf16 is None and self.resident:
            return                               # on the CPU the working copy is the fp32 arena
        _materialise(m)
        with torch.no_grad():
            for r in self.ranges:
                if r.size > 1:
                    dist.all_gather_into_tensor(m[r.start:r.end], r.own_master, group=r.group)
                else:
                    m[r.start:r.end].copy_(r.own_master)
        if self.arena.bf16 is None:
            self.resident = True

    def adopt_masters(self) -> None:
        """Take this rank's slices from the (edited) full fp32 values."""
        with torch.no_grad():
            for r in self.ranges:
                r.own_master.copy_(self.arena.master[r.lo:r.hi])
                if r.own_work is not None:
                    r.own_work.copy_(r.own_master)

    def release_masters(self) -> None:
        if self.arena.bf16 is None:
            self.release()
        else:
            _free(self.arena.master)

    def owned_numel(self) -> int:
        return sum(r.per for r in self.ranges)

    def resident_bytes(self) -> int:
        a = self.arena
        return sum(t.untyped_storage().size() for t in (a.master, a.grad, a.bf16) if t is not None)


def transformer_block_groups(model, blocks_per_unit: int = 1) -> List[Tuple[str, List[torch.nn.Module]]]:
    """Consecutive blocks of every ``BasicLayer`` (any module with a ``blocks`` list), ``blocks_per_unit`` at a time."""
    out = []
    for lname, layer in model.named_modules():
        blocks = getattr(layer, "blocks", None)
        if not isinstance(blocks, torch.nn.ModuleList):
            continue
        items = list(blocks)
        for s in range(0, len(items), max(1, int(blocks_per_unit))):
            out.append((f"{lname or 'model'}.blocks[{s}:{min(len(items), s + blocks_per_unit)}]", items[s:s + blocks_per_unit]))
    return out


class ParamSharder:
    """Owns the units of one model and the hooks that gather and release them."""

    def __init__(self, model: torch.nn.Module, resolve_group: Optional[Callable] = None, blocks_per_unit: int = 1,
                 whole_model: bool = False, prefetch: str = "none", reshard_after_forward: bool = True,
                 sampling_units: bool = False, bf16_shadow: Optional[bool] = None):
        """``bf16_shadow``: keep a bf16 working copy next to the fp32 values (default: on CUDA only); it is then the copy
        that is gathered, and the fp32 values exist only under ``summon_full_params``."""
        prefetch = (prefetch or "none").lower()
        if prefetch not in PREFETCH_POLICIES:
            raise ValueError(f"Unsupported FSDP prefetch policy: {prefetch}")
        self.model = model
        self.bf16_shadow = bf16_shadow
        self.prefetch = prefetch
        self.reshard_after_forward = bool(reshard_after_forward)
        resolve = resolve_group or (lambda label: (None, 0, 1))
        names = {id(p): n for n, p in model.named_parameters()}
        self.param_order = [p for p in model.parameters()]
        taken = set()
        self.units: List[ShardedUnit] = []
        self._reducing_unit: Optional[ShardedUnit] = None
        self._hooks = []
        groups = [] if whole_model else transformer_block_groups(model, blocks_per_unit)
        self.named_units: Dict[int, ShardedUnit] = {}          # id(module) -> unit, for run_in_unit
        self._depth: Dict[int, int] = {}
        head, tail = [], []
        if sampling_units and not whole_model:
            for attr, where in (("patch_embed", head), ("down_blk", head), ("up_blk", tail), ("patch_recovery", tail)):
                mod = getattr(model, attr, None)
                if isinstance(mod, torch.nn.Module) and any(p.requires_grad for p in mod.parameters()):
                    where.append((attr, mod))
        for attr, mod in head:
            self._add_function_unit(attr, mod, names, taken, resolve)
        for uname, mods in groups:
            ps = []
            for m in mods:
                for p in m.parameters():
                    if id(p) not in taken and p.requires_grad:
                        taken.add(id(p))
                        ps.append((names[id(p)], p))
            if not ps:
                continue
            sub = [x for m in mods for x in m.modules()]
            unit = ShardedUnit(uname, model, ps, sub, resolve, len(self.units), bf16_shadow)
            self.units.append(unit)
            self._hooks.append(mods[0].register_forward_pre_hook(lambda mod, args, u=unit: self._pre_forward(u)))
            for m in mods:
                last = m is mods[-1]
                self._hooks.append(m.register_forward_hook(lambda mod, args, out, u=unit, last=last: self._post_forward(u, out, last)))
        for attr, mod in tail:
            self._add_function_unit(attr, mod, names, taken, resolve)
        rest = [(n, p) for n, p in model.named_parameters() if id(p) not in taken and p.requires_grad]
        frozen = [n for n, p in model.named_parameters() if not p.requires_grad]
        if frozen:
            raise ValueError(f"parameter sharding needs every parameter trainable; frozen: {frozen[:3]}")
        self.root: Optional[ShardedUnit] = None
        if rest:
            covered = {id(x) for u_, mods in groups for m in mods for x in m.modules()}
            covered |= {id(x) for _, mod in head + tail for x in mod.modules()}
            sub = [m for m in model.modules() if id(m) not in covered]
            self.root = ShardedUnit("root", model, rest, sub, resolve, -1, bf16_shadow)
            self._hooks.append(model.register_forward_pre_hook(lambda mod, args: self._root_pre_forward()))
        model._param_sharder = self
        model.pre_wrap_parameter_count = sum(p.numel() for p in self.param_order)

    def _add_function_unit(self, name, mod, names, taken, resolve):
        ps = [(names[id(p)], p) for p in mod.parameters() if id(p) not in taken and p.requires_grad]
        for _, p in ps:
            taken.add(id(p))
        unit = ShardedUnit(name, self.model, ps, list(mod.modules()), resolve, len(self.units), self.bf16_shadow)
        self.units.append(unit)
        self.named_units[id(mod)] = unit
        self._depth[id(mod)] = 0

    def run_in_unit(self, mod: torch.nn.Module, fn: Callable, *args):
        """``fn(*args)`` with the unit of ``mod`` resident; calls may nest (a block function calling its layers'
        functions): the outermost one gathers and releases."""
        unit = self.named_units.get(id(mod))
        if unit is None:
            return fn(*args)
        key = id(mod)
        if self._depth[key] == 0:
            self._pre_forward(unit)
        self._depth[key] += 1
        try:
            out = fn(*args)
        finally:
            self._depth[key] -= 1
        self._post_forward(unit, out, last=self._depth[key] == 0)
        return out

    # ------------------------------------------------------------------ schedule
    def all_units(self) -> List[ShardedUnit]:
        return self.units + ([self.root] if self.root is not None else [])

    def _root_pre_forward(self):
        self.root.gather()
        if torch.is_grad_enabled():
            self.root.materialise_grad()

    def _neighbour(self, unit: ShardedUnit, step: int) -> Optional[ShardedUnit]:
        i = unit.index + step
        return self.units[i] if 0 <= i < len(self.units) else None

    def _pre_forward(self, unit: ShardedUnit):
        unit.gather()
        if self.prefetch == "overlap" and not _inside_backward():
            nxt = self._neighbour(unit, +1)
            if nxt is not None:
                nxt.gather(async_op=True)

    def _post_forward(self, unit: ShardedUnit, out, last: bool):
        if torch.is_grad_enabled():
            for t in (out if isinstance(out, (tuple, list)) else (out,)):
                if isinstance(t, torch.Tensor) and t.requires_grad:
                    t.register_hook(lambda g, u=unit: self._pre_backward(u))
        if not last or unit.in_backward or _inside_backward() or not self.reshard_after_forward:
            return
        unit.release()

    def _pre_backward(self, unit: ShardedUnit):
        for u in self.units:
            if u.in_backward and u is not unit:
                self._leave_backward(u)
        unit.gather()
        unit.materialise_grad()
        unit.in_backward = True
        if self.prefetch == "overlap":
            prv = self._neighbour(unit, -1)
            if prv is not None:
                prv.gather(async_op=True)
        return None

    def _leave_backward(self, unit: ShardedUnit):
        overlap = self.prefetch == "overlap"
        if self._reducing_unit is not None and self._reducing_unit is not unit:
            self._reducing_unit.finish_reduce()       # at most one unit's reduction in flight besides the new one
        unit.reduce_grad(async_op=overlap)
        self._reducing_unit = unit if overlap else None
        unit.release()
        unit.in_backward = False

    def finish_backward(self) -> None:
        """Collective. Reduce and release whatever the backward pass left: the unit it ended in, gradients that
        arrived after their unit had been left, and the root."""
        for u in self.units:
            if u.in_backward:
                self._leave_backward(u)
            elif u.has_stray_gradients():
                u.materialise_grad()
                u.reduce_grad()
            if u.resident:
                u.release()
        for u in self.units:
            u.finish_reduce()
        self._reducing_unit = None
        if self.root is not None:
            if self.root.has_stray_gradients():
                self.root.materialise_grad()
            self.root.reduce_grad()
            self.root.release()

    def zero_grad(self) -> None:
        for u in self.all_units():
            if u.grad_live:
                u.arena.grad.zero_()
            for r in u.ranges:
                r.own_grad.zero_()

    # ------------------------------------------------------------------ whole-model access
    @contextlib.contextmanager
    def summon_full_params(self, writeback: bool = False):
        """Collective. Inside, every parameter's ``.data`` holds its full fp32 value (``state_dict`` / ``load_state_dict``
        work as on an unsharded model); with ``writeback`` the owned slices are taken from the edited values on exit."""
        units = self.all_units()
        for u in units:
            u.gather_masters()
        try:
            yield self.model
        finally:
            for u in units:
                if writeback:
                    u.adopt_masters()
                u.release_masters()

    def full_state_dict(self) -> Dict[str, torch.Tensor]:
        with self.summon_full_params():
            return {k: v.detach().cpu().clone() for k, v in self.model.state_dict().items()}

    def load_full_state_dict(self, state, strict: bool = True):
        with self.summon_full_params(writeback=True):
            return self.model.load_state_dict(state, strict=strict)

    # ------------------------------------------------------------------ reports
    def owned_numel(self) -> int:
        return sum(u.owned_numel() for u in self.all_units())

    def total_numel(self) -> int:
        return sum(u.arena.numel for u in self.all_units())

    def resident_bytes(self) -> int:
        return sum(u.resident_bytes() for u in self.all_units())

    def describe(self) -> str:
        sizes = sorted({r.size for u in self.all_units() for r in u.ranges})
        return (f"[param sharding] units={len(self.units)} (+root={self.root is not None}), "
                f"elements total={self.total_numel()} owned={self.owned_numel()}, group sizes={sizes}, "
                f"prefetch_policy={self.prefetch}")

    def observe_gradients(self, callback) -> None:
        """``callback(unit)`` runs for every unit just before its gradients are reduce-scattered."""
        for u in self.all_units():
            u.gradient_observer = callback

    def remove_hooks(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks = []


def get_sharder(model) -> Optional[ParamSharder]:
    real = model.module if hasattr(model, "module") else model
    return getattr(real, "_param_sharder", None)
