"""CUDA memory timeline: per-iteration records of allocator state at named phases.

Keeps the reference's surface (profiler/memory_timeline.py:11-58,129-151,172-727): a context manager per
iteration, ``mark(phase, label, **meta)`` from the step runtime and from model code, identity autograd nodes
that mark when backward crosses a primitive boundary, per-primitive interval peaks keyed by ``occurrence_id``,
CSV / summary output, capture windows selected by ``MEMORY_TIMELINE_*`` environment variables.
Plotting is optional (matplotlib ``Agg`` when installed).
"""
from __future__ import annotations

import csv
import os
import threading
import time
from collections import defaultdict
from typing import Any, Dict, List, Optional

import torch

_ACTIVE: Optional["CudaMemoryTimeline"] = None
_CONTEXT: Dict[str, Any] = {}
_OCCURRENCES: Dict[str, int] = defaultdict(int)
_LOCK = threading.Lock()


def _env_int(name, default):
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def _env_flag(name, default="0"):
    return os.environ.get(name, default).strip().lower() in ("1", "true", "yes", "on")


MEMORY_TIMELINE_OUTPUT_START_ITER = _env_int("MEMORY_TIMELINE_OUTPUT_START_ITER", 0)
MEMORY_TIMELINE_OUTPUT_MAX_ITERS = _env_int("MEMORY_TIMELINE_OUTPUT_MAX_ITERS", 4)
MEMORY_TIMELINE_SYNC = _env_flag("MEMORY_TIMELINE_SYNC", "0")
MEMORY_TIMELINE_PLOT = _env_flag("MEMORY_TIMELINE_PLOT", "0")
MEMORY_TIMELINE_MODULE_HOOKS = _env_flag("MEMORY_TIMELINE_MODULE_HOOKS", "0")
MEMORY_TIMELINE_MAX_EVENTS = _env_int("MEMORY_TIMELINE_MAX_EVENTS", 200000)


def get_memory_timeline_context() -> Dict[str, Any]:
    return dict(_CONTEXT)


def set_memory_timeline_context(**kw) -> None:
    _CONTEXT.update(kw)


def new_memory_timeline_occurrence(primitive_id: str) -> str:
    with _LOCK:
        _OCCURRENCES[primitive_id] += 1
        return f"{primitive_id}#{_OCCURRENCES[primitive_id]}"


def mark_memory_timeline(phase: str, label: str = "", **meta) -> None:
    """No-op unless a timeline is active for the current iteration."""
    tl = _ACTIVE
    if tl is not None:
        tl.mark(phase, label, **meta)


class _BackwardMark(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, phase, label, meta):
        ctx.p = (phase, label, meta)
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        phase, label, meta = ctx.p
        mark_memory_timeline(phase, label, **meta)
        return g, None, None, None


def profile_memory_backward_boundary(x, phase, label, **meta):
    """Identity in forward; emits ``phase`` when backward passes through (exact backward boundaries)."""
    if _ACTIVE is None or not torch.is_tensor(x) or not x.requires_grad:
        return x
    return _BackwardMark.apply(x, phase, label, meta)


class CudaMemoryTimeline:
    FIELDS = ["iter", "seq", "time_s", "phase", "label", "allocated_mib", "reserved_mib", "max_allocated_mib",
              "driver_used_mib", "external_mib", "meta"]

    def __init__(self, device=None, enabled=True, output_dir=None, tag="rank0"):
        self.device = device
        self.enabled = enabled and torch.cuda.is_available()
        self.force_cpu = enabled and not torch.cuda.is_available()
        self.output_dir = output_dir
        self.tag = tag
        self.events: List[Dict[str, Any]] = []
        self.iter_idx = -1
        self._seq = 0
        self._t0 = time.time()
        self._hooks = []

    # ---- iteration scope
    def iteration(self, iter_idx: int):
        self.iter_idx = iter_idx
        return self

    def __enter__(self):
        global _ACTIVE
        start = MEMORY_TIMELINE_OUTPUT_START_ITER
        in_window = start <= self.iter_idx < start + MEMORY_TIMELINE_OUTPUT_MAX_ITERS
        if (self.enabled or self.force_cpu) and in_window:
            _ACTIVE = self
            if self.enabled:
                torch.cuda.reset_peak_memory_stats(self.device)
            self.mark("iter_start", "")
        return self

    def __exit__(self, *exc):
        global _ACTIVE
        if _ACTIVE is self:
            self.mark("iter_end", "")
            _ACTIVE = None
        return False

    # ---- records
    def _snapshot(self):
        if not self.enabled:
            return 0.0, 0.0, 0.0, 0.0, 0.0
        if MEMORY_TIMELINE_SYNC:
            torch.cuda.synchronize(self.device)
        mib = 1.0 / (1 << 20)
        alloc = torch.cuda.memory_allocated(self.device) * mib
        reserved = torch.cuda.memory_reserved(self.device) * mib
        peak = torch.cuda.max_memory_allocated(self.device) * mib
        free, total = torch.cuda.mem_get_info(self.device)
        used = (total - free) * mib
        return alloc, reserved, peak, used, max(0.0, used - reserved)

    def mark(self, phase, label="", **meta):
        if len(self.events) >= MEMORY_TIMELINE_MAX_EVENTS:
            return
        alloc, reserved, peak, used, ext = self._snapshot()
        self._seq += 1
        self.events.append(dict(iter=self.iter_idx, seq=self._seq, time_s=time.time() - self._t0, phase=phase,
                                label=label, allocated_mib=alloc, reserved_mib=reserved, max_allocated_mib=peak,
                                driver_used_mib=used, external_mib=ext, meta=dict(meta)))

    # ---- module hooks (optional)
    def attach(self, model: torch.nn.Module, depth: int = 2):
        if not MEMORY_TIMELINE_MODULE_HOOKS:
            return
        for name, mod in model.named_modules():
            if name and name.count(".") < depth:
                self._hooks.append(mod.register_forward_pre_hook(lambda m, i, n=name: self.mark("module_fwd_pre", n)))
                self._hooks.append(mod.register_forward_hook(lambda m, i, o, n=name: self.mark("module_fwd_post", n)))
                self._hooks.append(mod.register_full_backward_hook(lambda m, gi, go, n=name: self.mark("module_bwd_post", n)))

    def detach(self):
        for h in self._hooks:
            h.remove()
        self._hooks = []

    # ---- analysis
    def primitive_intervals(self) -> List[Dict[str, Any]]:
        """Peak-memory rise between the pre/post marks of every primitive occurrence, forward and backward."""
        opened: Dict[Any, Dict[str, Any]] = {}
        rows = []
        pairs = {"primitive_forward_pre": ("primitive_forward_post", "forward"),
                 "primitive_backward_pre": ("primitive_backward_post", "backward")}
        closing = {v[0]: (k, v[1]) for k, v in pairs.items()}
        for i, ev in enumerate(self.events):
            occ = ev["meta"].get("occurrence_id")
            if occ is None:
                continue
            if ev["phase"] in pairs:
                opened[(occ, pairs[ev["phase"]][1])] = dict(start=i, base=ev["allocated_mib"])
            elif ev["phase"] in closing:
                direction = closing[ev["phase"]][1]
                st = opened.pop((occ, direction), None)
                if st is None:
                    continue
                peak = max(e["allocated_mib"] for e in self.events[st["start"]:i + 1])
                rows.append(dict(iter=ev["iter"], occurrence_id=occ, direction=direction,
                                 primitive_kind=ev["meta"].get("primitive_kind", ""),
                                 primitive_id=ev["meta"].get("primitive_id", ""), lead_idx=ev["meta"].get("lead_idx", ""),
                                 base_mib=st["base"], interval_peak_mib=peak, interval_peak_rise_mib=peak - st["base"],
                                 end_mib=ev["allocated_mib"]))
        return rows

    def summary(self) -> Dict[str, Any]:
        by_iter: Dict[int, float] = defaultdict(float)
        for ev in self.events:
            by_iter[ev["iter"]] = max(by_iter[ev["iter"]], ev["max_allocated_mib"], ev["allocated_mib"])
        return {"iters": sorted(by_iter), "peak_allocated_mib": dict(by_iter), "num_events": len(self.events)}

    # ---- output
    def write_csv(self, path: str) -> None:
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=self.FIELDS)
            w.writeheader()
            for ev in self.events:
                row = dict(ev)
                row["meta"] = ";".join(f"{k}={v}" for k, v in sorted(ev["meta"].items()))
                w.writerow(row)

    def write_summary_csv(self, path: str) -> None:
        rows = self.primitive_intervals()
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "w", newline="") as f:
            fields = ["iter", "occurrence_id", "direction", "primitive_kind", "primitive_id", "lead_idx", "base_mib",
                      "interval_peak_mib", "interval_peak_rise_mib", "end_mib"]
            w = csv.DictWriter(f, fieldnames=fields)
            w.writeheader()
            for r in rows:
                w.writerow(r)

    def plot(self, path: str) -> bool:
        try:
            import matplotlib

            matplotlib.use("Agg")
            import matplotlib.pyplot as plt
        except Exception:
            return False
        fig, ax = plt.subplots(figsize=(12, 4))
        ax.plot([e["seq"] for e in self.events], [e["allocated_mib"] for e in self.events], label="allocated")
        ax.plot([e["seq"] for e in self.events], [e["reserved_mib"] for e in self.events], label="reserved")
        ax.set_xlabel("event")
        ax.set_ylabel("MiB")
        ax.legend()
        fig.savefig(path, dpi=120)
        plt.close(fig)
        return True
