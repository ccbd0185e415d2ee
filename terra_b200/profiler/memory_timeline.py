"""CUDA memory timeline: per-iteration records of allocator state at named phases.

Keeps the reference's surface (profiler/memory_timeline.py:11-58,129-151,172-727): a context manager per
iteration, ``mark(phase, label, **meta)`` from the step runtime and from model code, identity autograd nodes
that mark when backward crosses a primitive boundary, per-primitive interval peaks keyed by ``occurrence_id``,
true allocator peaks of measured intervals (the peak counter is restarted at every interval opener and the peaks folded
away are kept for ``get_memory_timeline_peak_mib``), CSV / summary / event-table / plot output, capture windows and
plot filters selected by ``MEMORY_TIMELINE_*`` environment variables. Plotting is optional (matplotlib ``Agg`` when
installed).
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
# what write_outputs() produces, and what the plot / the event table show (reference switches of the same names,
# profiler/memory_timeline.py:11-37)
MEMORY_TIMELINE_WRITE_CSV = _env_flag("MEMORY_TIMELINE_WRITE_CSV", "1")
MEMORY_TIMELINE_WRITE_SUMMARY = _env_flag("MEMORY_TIMELINE_WRITE_SUMMARY", "1")
MEMORY_TIMELINE_WRITE_EVENT_TABLE = _env_flag("MEMORY_TIMELINE_WRITE_EVENT_TABLE", "1")
MEMORY_TIMELINE_WRITE_PLOT = _env_flag("MEMORY_TIMELINE_WRITE_PLOT", "1")
MEMORY_TIMELINE_ANNOTATE_EVENTS = _env_flag("MEMORY_TIMELINE_ANNOTATE_EVENTS", "1")
MEMORY_TIMELINE_MAX_EVENT_ANNOTATIONS = _env_int("MEMORY_TIMELINE_MAX_EVENT_ANNOTATIONS", 120)
MEMORY_TIMELINE_X_AXIS = os.environ.get("MEMORY_TIMELINE_X_AXIS", "time").strip().lower()      # "time" | "event"
MEMORY_TIMELINE_SHOW_MODULE_HOOKS = _env_flag("MEMORY_TIMELINE_SHOW_MODULE_HOOKS", "0")
MEMORY_TIMELINE_SHOW_SAMPLING_INTERNALS = _env_flag("MEMORY_TIMELINE_SHOW_SAMPLING_INTERNALS", "0")
MEMORY_TIMELINE_SHOW_CHECKPOINT_BODY = _env_flag("MEMORY_TIMELINE_SHOW_CHECKPOINT_BODY", "0")

# ---- event classes: what a phase name means for the plot and the event table
COARSE_PHASES = ("iter_start", "before_forward", "after_forward", "before_backward", "after_backward", "before_optimizer",
                 "after_optimizer", "iter_end")
SAMPLING_BOUNDARY_PHASES = ("sampling_down_enter", "sampling_down_exit", "sampling_up_enter", "sampling_up_exit")
INTERVAL_PAIRS = {                      # opener -> (closer, kind): the allocator peak is measured between the two
    "primitive_forward_pre": ("primitive_forward_post", "primitive_forward"),
    "primitive_backward_pre": ("primitive_backward_post", "primitive_backward"),
    "checkpoint_edge_pre": ("checkpoint_edge_post", "checkpoint_edge"),
    "transformer_segment_pre": ("transformer_segment_post", "transformer_segment"),
    "transformer_segment_checkpoint_pre": ("transformer_segment_checkpoint_post", "transformer_segment_checkpoint"),
}
_INTERVAL_CLOSERS = {closer: (opener, kind) for opener, (closer, kind) in INTERVAL_PAIRS.items()}
CHECKPOINT_BOUNDARY_PHASES = tuple(INTERVAL_PAIRS) + tuple(_INTERVAL_CLOSERS)


def event_class(phase: str) -> str:
    """``coarse`` (step phases), ``sampling_boundary``, ``checkpoint_boundary`` (segment / primitive edges),
    ``module_hook``, ``sampling_internal`` (marks inside the down / up blocks), ``checkpoint_body`` (marks emitted while a
    checkpointed segment recomputes) or ``other``."""
    if phase in COARSE_PHASES:
        return "coarse"
    if phase in SAMPLING_BOUNDARY_PHASES:
        return "sampling_boundary"
    if phase in CHECKPOINT_BOUNDARY_PHASES:
        return "checkpoint_boundary"
    if phase.startswith("module_"):
        return "module_hook"
    if phase.startswith("sampling_"):
        return "sampling_internal"
    if phase.startswith("recompute_") or phase.startswith("checkpoint_body"):
        return "checkpoint_body"
    return "other"


def event_visible(phase: str) -> bool:
    """Whether the plot and the event table show an event of this phase (the CSV always holds every event)."""
    cls = event_class(phase)
    if cls == "module_hook":
        return MEMORY_TIMELINE_SHOW_MODULE_HOOKS
    if cls == "sampling_internal":
        return MEMORY_TIMELINE_SHOW_SAMPLING_INTERNALS
    if cls == "checkpoint_body":
        return MEMORY_TIMELINE_SHOW_CHECKPOINT_BODY
    return True


def memory_timeline_iteration_enabled(iter_idx: int) -> bool:
    """Whether this iteration lies inside the capture window ``[START_ITER, START_ITER + MAX_ITERS)``."""
    start = MEMORY_TIMELINE_OUTPUT_START_ITER
    return MEMORY_TIMELINE_OUTPUT_MAX_ITERS > 0 and start <= int(iter_idx) < start + MEMORY_TIMELINE_OUTPUT_MAX_ITERS


def get_memory_timeline_peak_mib() -> float:
    """Run-wide peak of allocated memory. The timeline resets the allocator's peak counter at the start of every
    measured interval, so ``torch.cuda.max_memory_allocated`` alone under-reports while one is active: the peaks folded
    away at each reset are kept by the timeline."""
    if not torch.cuda.is_available():
        return 0.0
    now = torch.cuda.max_memory_allocated() / (1 << 20)
    tl = _ACTIVE
    return now if tl is None else max(now, tl.overall_peak_allocated_mib)


def get_memory_timeline_context() -> Dict[str, Any]:
    return dict(_CONTEXT)


def set_memory_timeline_context(**kw) -> None:
    """Semantic context copied into every later event (``lead_idx``, ``execution_phase``, ...); ``None`` removes a key."""
    for k, v in kw.items():
        if v is None:
            _CONTEXT.pop(k, None)
        else:
            _CONTEXT[k] = v


def new_memory_timeline_occurrence(primitive_id: str) -> str:
    with _LOCK:
        _OCCURRENCES[primitive_id] += 1
        return f"{primitive_id}#{_OCCURRENCES[primitive_id]}"


def mark_memory_timeline(phase: str, label: str = "", **meta) -> None:
    """No-op unless a timeline is active for the current iteration."""
    tl = _ACTIVE
    if tl is not None:
        merged = dict(_CONTEXT)
        merged.update(meta)
        tl.mark(phase, label, **merged)


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
        self.overall_peak_allocated_mib = 0.0      # peaks folded away by the interval resets (see _fold_peak_and_reset)
        self.iteration_peak_allocated_mib = 0.0    # the same, restarted at every iteration (read it after the step)
        self._open: Dict[Any, float] = {}            # (interval kind, occurrence or label) -> allocated MiB at the opener

    # ---- iteration scope
    def iteration(self, iter_idx: int):
        self.iter_idx = iter_idx
        return self

    def __enter__(self):
        global _ACTIVE
        if (self.enabled or self.force_cpu) and memory_timeline_iteration_enabled(self.iter_idx):
            _ACTIVE = self
            self._fold_peak_and_reset()
            self.iteration_peak_allocated_mib = 0.0
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

    def _fold_peak_and_reset(self) -> None:
        """Keep the allocator's peak so far in ``overall_peak_allocated_mib`` and restart its peak counter, so that
        the next read of ``max_memory_allocated`` is the peak of the interval that starts here."""
        if not self.enabled:
            return
        seen = torch.cuda.max_memory_allocated(self.device) / (1 << 20)
        self.overall_peak_allocated_mib = max(self.overall_peak_allocated_mib, seen)
        self.iteration_peak_allocated_mib = max(self.iteration_peak_allocated_mib, seen)
        torch.cuda.reset_peak_memory_stats(self.device)

    def _interval_meta(self, phase, label, meta, alloc, peak) -> Dict[str, Any]:
        """Open / close the measured interval this event belongs to. The closer's record carries the interval's start
        level, its true allocator peak (transient allocations between two marks included) and the rise."""
        key_of = lambda kind: (kind, meta.get("occurrence_id") or label)
        if phase in INTERVAL_PAIRS:
            self._open[key_of(INTERVAL_PAIRS[phase][1])] = alloc
            self._fold_peak_and_reset()
            return {}
        if phase in _INTERVAL_CLOSERS:
            kind = _INTERVAL_CLOSERS[phase][1]
            start = self._open.pop(key_of(kind), None)
            if start is None:
                return {}
            top = max(peak, alloc, start)
            return {"interval_kind": kind, "interval_start_allocated_mib": start, "interval_peak_allocated_mib": top,
                    "interval_peak_rise_mib": top - start}
        return {}

    def mark(self, phase, label="", **meta):
        if len(self.events) >= MEMORY_TIMELINE_MAX_EVENTS:
            return
        alloc, reserved, peak, used, ext = self._snapshot()
        meta = dict(meta)
        meta.update(self._interval_meta(phase, label, meta, alloc, peak))
        self.overall_peak_allocated_mib = max(self.overall_peak_allocated_mib, peak, alloc)
        self.iteration_peak_allocated_mib = max(self.iteration_peak_allocated_mib, peak, alloc)
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
                peak = max(peak, float(ev["meta"].get("interval_peak_allocated_mib", 0.0) or 0.0))   # allocator peak, when measured
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
        out = {"iters": sorted(by_iter), "peak_allocated_mib": dict(by_iter), "num_events": len(self.events),
               "overall_peak_allocated_mib": max([self.overall_peak_allocated_mib] + list(by_iter.values()))}
        # where every metric peaks: the event (phase, label, iteration) at which it was highest
        for key in ("allocated_mib", "reserved_mib", "driver_used_mib", "external_mib"):
            if self.events:
                top = max(self.events, key=lambda e: e[key])
                out["max_" + key] = {"value": top[key], "iter": top["iter"], "phase": top["phase"], "label": top["label"]}
        return out

    def visible_events(self) -> List[Dict[str, Any]]:
        return [e for e in self.events if event_visible(e["phase"])]

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

    def write_event_table(self, path: str) -> None:
        """Fixed-width text table of the visible events, one line each, with the change of allocated memory since the
        previous line: the file to read next to the plot (reference: profiler/memory_timeline.py:562-588)."""
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        rows = self.visible_events()
        with open(path, "w") as f:
            f.write(f"{'seq':>6} {'iter':>5} {'time_s':>9} {'class':<20} {'phase':<38} {'label':<30} "
                    f"{'alloc MiB':>11} {'delta':>10} {'reserved':>10} {'peak':>10}  interval\n")
            prev = None
            for e in rows:
                delta = 0.0 if prev is None else e["allocated_mib"] - prev
                prev = e["allocated_mib"]
                m = e["meta"]
                interval = ""
                if "interval_kind" in m:
                    interval = (f"{m['interval_kind']} start {m['interval_start_allocated_mib']:.1f} "
                                f"peak {m['interval_peak_allocated_mib']:.1f} rise {m['interval_peak_rise_mib']:+.1f}")
                f.write(f"{e['seq']:>6} {e['iter']:>5} {e['time_s']:>9.4f} {event_class(e['phase']):<20} {e['phase'][:38]:<38} "
                        f"{str(e['label'])[:30]:<30} {e['allocated_mib']:>11.1f} {delta:>+10.1f} {e['reserved_mib']:>10.1f} "
                        f"{e['max_allocated_mib']:>10.1f}  {interval}\n")

    def write_summary(self, path: str) -> None:
        """``key: value`` lines of ``summary()`` (peaks per iteration, where each metric peaks, the run-wide peak)."""
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        sm = self.summary()
        with open(path, "w") as f:
            f.write(f"events: {sm['num_events']}\noverall_peak_allocated_mib: {sm['overall_peak_allocated_mib']:.1f}\n")
            for it in sm["iters"]:
                f.write(f"iter {it} peak_allocated_mib: {sm['peak_allocated_mib'][it]:.1f}\n")
            for key in ("allocated_mib", "reserved_mib", "driver_used_mib", "external_mib"):
                top = sm.get("max_" + key)
                if top is not None:
                    f.write(f"max {key}: {top['value']:.1f} at iter {top['iter']} {top['phase']} {top['label']}\n")

    def write_outputs(self, output_dir: Optional[str] = None, tag: Optional[str] = None) -> Dict[str, str]:
        """Everything the ``MEMORY_TIMELINE_WRITE_*`` switches ask for, under ``output_dir``; returns the paths."""
        d = output_dir or self.output_dir or os.environ.get("MEMORY_TIMELINE_OUTPUT_DIR", "./log/memory_timeline")
        tag = tag or self.tag
        made = {}
        if not self.events:
            return made
        if MEMORY_TIMELINE_WRITE_CSV:
            made["csv"] = os.path.join(d, f"timeline_{tag}.csv")
            self.write_csv(made["csv"])
        if MEMORY_TIMELINE_WRITE_SUMMARY:
            made["summary"] = os.path.join(d, f"summary_{tag}.txt")
            self.write_summary(made["summary"])
            made["primitive_summary"] = os.path.join(d, f"primitive_summary_{tag}.csv")
            self.write_summary_csv(made["primitive_summary"])
        if MEMORY_TIMELINE_WRITE_EVENT_TABLE:
            made["event_table"] = os.path.join(d, f"events_{tag}.txt")
            self.write_event_table(made["event_table"])
        if MEMORY_TIMELINE_WRITE_PLOT and self.plot(os.path.join(d, f"timeline_{tag}.png")):
            made["plot"] = os.path.join(d, f"timeline_{tag}.png")
        return made

    def plot(self, path: str) -> bool:
        """Allocated / reserved memory over time (or over the event index, ``MEMORY_TIMELINE_X_AXIS=event``) for the
        visible events; step phases as vertical lines, segment and sampling boundaries annotated up to
        ``MEMORY_TIMELINE_MAX_EVENT_ANNOTATIONS``. Returns False when matplotlib is not installed."""
        try:
            import matplotlib

            matplotlib.use("Agg")
            import matplotlib.pyplot as plt
        except Exception:
            return False
        rows = self.visible_events()
        if not rows:
            return False
        by_event = MEMORY_TIMELINE_X_AXIS == "event"
        xs = [i if by_event else e["time_s"] for i, e in enumerate(rows)]
        fig, ax = plt.subplots(figsize=(14, 5))
        ax.plot(xs, [e["allocated_mib"] for e in rows], label="allocated", linewidth=1.2)
        ax.plot(xs, [e["reserved_mib"] for e in rows], label="reserved", linewidth=0.8, alpha=0.7)
        ax.plot(xs, [e["max_allocated_mib"] for e in rows], label="allocator peak since last reset", linewidth=0.6, alpha=0.6)
        notes = 0
        for x, e in zip(xs, rows):
            cls = event_class(e["phase"])
            if cls == "coarse":
                ax.axvline(x, color="0.8", linewidth=0.5)
            if MEMORY_TIMELINE_ANNOTATE_EVENTS and notes < MEMORY_TIMELINE_MAX_EVENT_ANNOTATIONS and cls in (
                    "coarse", "sampling_boundary", "checkpoint_boundary"):
                text = e["phase"] if not e["label"] else f"{e['phase']}:{e['label']}"
                ax.annotate(text[:28], (x, e["allocated_mib"]), fontsize=5, rotation=60, alpha=0.8)
                notes += 1
        ax.set_xlabel("event" if by_event else "seconds")
        ax.set_ylabel("MiB")
        ax.legend(fontsize=7)
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        fig.savefig(path, dpi=130)
        plt.close(fig)
        return True
