"""Flat parameter arenas.

All parameters of a model are re-pointed into three flat buffers:

* ``master``  fp32 - the values the optimizer updates (``p.data`` becomes a view),
* ``grad``    fp32 - ``p.grad`` becomes a view; the weight-gradient kernels accumulate into it directly,
* ``bf16``    the working copy the sm_100a kernels read (``p.bf16``), rewritten by the fused AdamW kernel.

Modules may declare ``_fused_param_groups = {"name": [param names...]}``: those parameters are laid out back to
back so that their concatenation along dim 0 is a free view (``module.fused["name"]``), e.g. the q/k/v
projection weights of an attention block form one ``[3C, C]`` GEMM operand while ``state_dict()`` still shows
three tensors. Arena segments are grouped by the communication label of the parameter
(``terra_grad_reduce_group``), so that gradient reduction and the sharded optimizer work on whole ranges.

The reference keeps ordinary per-parameter tensors: gradients are reduced parameter by parameter
(core/runtime/run_model.py:240-330), its ``DistributedAdamW`` assigns whole parameters to owners and broadcasts them
(optimizer/distributed_adamw.py:122-146, 202-264); the arenas are what lets one collective and one kernel do that work
here while the parameter names, shapes and ``state_dict`` stay the reference's.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

ALIGN = 64  # elements: 128 B in bf16, 256 B in fp32 -> every parameter is a legal TMA base
SEGMENT_ALIGN = ALIGN * 16  # a segment splits evenly over 1, 2, 4, 8 or 16 replica ranks in ALIGN-sized units


@dataclass
class FusedView:
    master: torch.Tensor
    grad: torch.Tensor
    bf16: Optional[torch.Tensor]


@dataclass
class Segment:
    label: str
    start: int
    end: int


def _label_of(p) -> str:
    return getattr(p, "terra_grad_reduce_group", None) or "full"


class ParamArena:
    def __init__(self, model: torch.nn.Module, bf16_shadow: Optional[bool] = None, params=None, modules=None,
                 segment_align: int = SEGMENT_ALIGN):
        """``params`` (a list of ``(name, parameter)``) and ``modules`` (where fused groups are looked up) restrict the
        arena to a part of ``model``, which then is not registered as the model's arena: the parameter-sharding units
        (``terra_b200.parallel.param_sharding``) each own one. ``segment_align``: every segment's length is a multiple
        of it (a multiple of ``ALIGN``; the default splits evenly over 1, 2, 4, 8 or 16 ranks)."""
        partial = params is not None
        params = [(n, p) for n, p in (model.named_parameters() if params is None else params)]
        if not params:
            raise ValueError("model has no parameters")
        if segment_align % ALIGN:
            raise ValueError(f"segment_align must be a multiple of {ALIGN}")
        wanted = {id(p) for _, p in params}
        device = params[0][1].device
        self.device = device
        self.bf16_shadow = (device.type == "cuda") if bf16_shadow is None else bf16_shadow

        # fused groups first (kept contiguous), then the rest, each bucketed by communication label
        name_of = {id(p): n for n, p in params}
        placed = set()
        ordered: Dict[str, List[Tuple[List[torch.nn.Parameter], Optional[Tuple[torch.nn.Module, str]]]]] = {}
        for mod in (model.modules() if modules is None else modules):
            groups = getattr(mod, "_fused_param_groups", None)
            if not groups:
                continue
            local = dict(mod.named_parameters())
            for gname, names in groups.items():
                members = [local[n] for n in names if n in local]
                if len(members) != len(names) or any(id(m) in placed or id(m) not in wanted for m in members):
                    continue
                labels = {_label_of(m) for m in members}
                if len(labels) != 1:
                    raise ValueError(f"fused group {gname} mixes communication labels {labels}")
                for m in members:
                    placed.add(id(m))
                ordered.setdefault(labels.pop(), []).append((members, (mod, gname)))
        for n, p in params:
            if id(p) not in placed:
                placed.add(id(p))
                ordered.setdefault(_label_of(p), []).append(([p], None))

        # layout
        offsets: Dict[int, int] = {}
        self.segments: List[Segment] = []
        cursor = 0
        for label in sorted(ordered):
            seg_start = cursor
            for members, _ in ordered[label]:
                cursor = (cursor + ALIGN - 1) // ALIGN * ALIGN
                for m in members:
                    offsets[id(m)] = cursor
                    cursor += m.numel()
            cursor = (cursor + segment_align - 1) // segment_align * segment_align
            self.segments.append(Segment(label, seg_start, cursor))
        self.numel = cursor

        self.master = torch.zeros(self.numel, dtype=torch.float32, device=device)
        self.grad = torch.zeros(self.numel, dtype=torch.float32, device=device)
        self.bf16 = torch.zeros(self.numel, dtype=torch.bfloat16, device=device) if self.bf16_shadow else None
        self.params: List[torch.nn.Parameter] = []
        self.names: List[str] = []
        self.offsets: List[int] = []
        for n, p in params:
            off = offsets[id(p)]
            view = self.master[off:off + p.numel()].view(p.shape)
            with torch.no_grad():
                view.copy_(p.data)
            p.data = view
            p.grad = self.grad[off:off + p.numel()].view(p.shape)
            p.bf16 = self.bf16[off:off + p.numel()].view(p.shape) if self.bf16 is not None else None
            p.arena_offset = off
            self.params.append(p)
            self.names.append(n)
            self.offsets.append(off)
        self._fused_records = []
        for label in ordered:
            for members, tag in ordered[label]:
                if tag is None:
                    continue
                mod, gname = tag
                off = offsets[id(members[0])]
                total = sum(m.numel() for m in members)
                shape = (sum(m.shape[0] for m in members),) + tuple(members[0].shape[1:])
                fused = getattr(mod, "fused", None)
                if fused is None:
                    fused = {}
                    mod.fused = fused
                self._fused_records.append((mod, gname, off, total, shape))
                fused[gname] = FusedView(
                    self.master[off:off + total].view(shape), self.grad[off:off + total].view(shape),
                    self.bf16[off:off + total].view(shape) if self.bf16 is not None else None)
        self.sync_bf16()
        if not partial:
            model._param_arena = self

    def rebind(self, grad: torch.Tensor, bf16: Optional[torch.Tensor]) -> None:
        """Move the gradient arena (and the bf16 working copy) into caller-provided flat buffers of the same
        length, e.g. peer-visible symmetric memory, and re-point every view."""
        if grad.numel() != self.numel or grad.dtype != torch.float32:
            raise ValueError("rebind: gradient buffer must be fp32 with the arena's length")
        grad.copy_(self.grad)
        self.grad = grad
        if bf16 is not None:
            if bf16.numel() != self.numel or bf16.dtype != torch.bfloat16:
                raise ValueError("rebind: working copy must be bf16 with the arena's length")
            bf16.copy_(self.master)
            self.bf16 = bf16
        for p, off in zip(self.params, self.offsets):
            p.grad = self.grad[off:off + p.numel()].view(p.shape)
            p.bf16 = self.bf16[off:off + p.numel()].view(p.shape) if self.bf16 is not None else None
        for mod, gname, off, total, shape in self._fused_records:
            mod.fused[gname] = FusedView(self.master[off:off + total].view(shape), self.grad[off:off + total].view(shape),
                                         self.bf16[off:off + total].view(shape) if self.bf16 is not None else None)

    def sync_bf16(self) -> None:
        """Refresh the bf16 working copy from the fp32 masters (after init or a checkpoint load)."""
        if self.bf16 is not None:
            self.bf16.copy_(self.master)
            from ..ops.conv import invalidate_packed_weights

            invalidate_packed_weights()

    def zero_grad(self) -> None:
        self.grad.zero_()
        for p, off in zip(self.params, self.offsets):
            if p.grad is None or p.grad.data_ptr() != self.grad.data_ptr() + off * 4:
                p.grad = self.grad[off:off + p.numel()].view(p.shape)

    def segment(self, label: str) -> Optional[Segment]:
        for s in self.segments:
            if s.label == label:
                return s
        return None


def get_arena(model) -> Optional[ParamArena]:
    return getattr(model, "_param_arena", None)
