"""Per-lead activation plans of rollout finetuning: which transformer segments are checkpointed (and how) and how the
sampling blocks are checkpointed may change from one lead of a rollout to the next, because later leads hold more
activations of earlier ones.

YAML (under ``activation:``; the formats of the reference harness, train_scripts/test_finetune.py:380-530, leads are
numbered from 1):

    lead_checkpoint_schedule:                 # also accepted under its older name lead_checkpoint_layers
      "1": []                                 # dict form: "<lead>" or "<first>-<last>" -> layer entries
      "2-3": ['0-3', 6]
      "4": {checkpoint_layers: ['0-7'], mode: cpu_boundary_offload_recompute, offload: {min_numel: 1048576}}
    lead_checkpoint_schedule:                 # list form, every field spelled out (aliases in brackets)
      - lead_start: 2                         # [start, lead]
        lead_end: 3                           # [end]; default: lead_start
        checkpoint_layers: "0-3, 6"           # [layers]; a list, or one string separated by commas / blanks
        activation_mode: torch_recompute      # [mode]; default: activation.mode
        segment_activation_modes: [torch_recompute, cpu_boundary_offload_recompute]   # one per entry; default: the mode
        offload: {min_numel: 1048576}         # default: activation.offload
        label: warm
    lead_sampling_checkpoint_schedule:
      "3-4": {down: D1, up: U1}               # or {sampling_checkpoint: {...}, sampling_modes: {down:, up:}, offload: {}}

A value that is itself a dict in the dict form of ``lead_checkpoint_schedule`` is read as a list-form entry (an
extension: the reference takes the value as the layer list only). The first entry whose range contains the lead wins;
entries are ordered by ``(lead_start, lead_end)``. A lead that no entry covers keeps the plan that is installed
(transformer) or returns to the base configuration (sampling), as in the reference.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from .activation import activation_config_for_sampling


def _lead_range(key) -> Tuple[int, int]:
    text = str(key).strip()
    if "-" in text:
        first, last = (part.strip() for part in text.split("-", 1))
        return int(first), int(last)
    return int(text), int(text)


def _words(value) -> List[str]:
    """A list as it is; one string cut at commas and blanks."""
    if isinstance(value, str):
        return [w for w in value.replace(",", " ").split() if w]
    return list(value)


def _entry_range(item: dict) -> Tuple[int, int]:
    first = int(item.get("lead_start", item.get("start", item.get("lead", 1))))
    return first, int(item.get("lead_end", item.get("end", first)))


@dataclass
class LeadPlan:
    lead_start: int
    lead_end: int
    checkpoint_layers: List[Any]
    activation_mode: str
    segment_activation_modes: List[str]
    offload: Dict[str, Any]
    label: str

    def covers(self, lead_number: int) -> bool:
        return self.lead_start <= lead_number <= self.lead_end


@dataclass
class LeadSamplingPlan:
    lead_start: int
    lead_end: int
    down: Optional[str]
    up: Optional[str]
    down_activation_mode: Optional[str]
    up_activation_mode: Optional[str]
    offload: Optional[Dict[str, Any]]
    label: str

    def covers(self, lead_number: int) -> bool:
        return self.lead_start <= lead_number <= self.lead_end


def parse_lead_checkpoint_schedule(activation: Optional[dict]) -> List[LeadPlan]:
    activation = activation or {}
    raw = activation.get("lead_checkpoint_schedule", activation.get("lead_checkpoint_layers"))
    if not raw:
        return []
    entries = []
    if isinstance(raw, dict):
        for key, value in raw.items():
            first, last = _lead_range(key)
            entry = dict(value) if isinstance(value, dict) else {"checkpoint_layers": value}
            entry.setdefault("lead_start", first)
            entry.setdefault("lead_end", last)
            entries.append(entry)
    else:
        entries = list(raw)
    plans = []
    for item in entries:
        if not isinstance(item, dict):
            raise ValueError(f"lead_checkpoint_schedule entries must be dicts, got: {item}")
        first, last = _entry_range(item)
        layers = item.get("checkpoint_layers", item.get("layers"))
        if layers is None:
            raise ValueError(f"lead_checkpoint_schedule entry missing checkpoint_layers: {item}")
        layers = _words(layers)
        mode = str(item.get("activation_mode", item.get("mode", activation.get("mode", "torch_recompute"))))
        seg = item.get("segment_activation_modes")
        seg = [mode] * len(layers) if seg is None else [str(m) for m in _words(seg)]
        if len(seg) != len(layers):
            raise ValueError("lead_checkpoint_schedule segment_activation_modes must match checkpoint_layers: "
                             f"{len(seg)} != {len(layers)} in {item}")
        offload = item.get("offload", activation.get("offload", {}))
        offload = {} if offload is None else offload
        if not isinstance(offload, dict):
            raise ValueError(f"lead_checkpoint_schedule offload must be a dict: {item}")
        plans.append(LeadPlan(first, last, layers, mode, seg, dict(offload), item.get("label", f"lead{first}-{last}")))
    return sorted(plans, key=lambda p: (p.lead_start, p.lead_end))


def parse_lead_sampling_schedule(activation: Optional[dict]) -> List[LeadSamplingPlan]:
    activation = activation or {}
    raw = activation.get("lead_sampling_checkpoint_schedule")
    if not raw:
        return []
    entries = []
    if isinstance(raw, dict):
        for key, value in raw.items():
            first, last = _lead_range(key)
            entry = dict(value or {}) if isinstance(value, dict) else {"sampling_checkpoint": value}
            entry["lead_start"], entry["lead_end"] = first, last
            entries.append(entry)
    else:
        entries = list(raw)
    plans = []
    for item in entries:
        if not isinstance(item, dict):
            raise ValueError(f"lead_sampling_checkpoint_schedule entries must be dicts, got: {item}")
        first, last = _entry_range(item)
        sampling = item.get("sampling_checkpoint", item.get("sampling", item))
        if not isinstance(sampling, dict):
            raise ValueError(f"lead_sampling_checkpoint_schedule entry missing sampling checkpoint dict: {item}")
        down, up = sampling.get("down"), sampling.get("up")
        if down is None and up is None:
            raise ValueError(f"lead_sampling_checkpoint_schedule entry must contain down or up: {item}")
        modes = item.get("sampling_modes") or {}
        if not isinstance(modes, dict):
            raise ValueError(f"lead_sampling_checkpoint_schedule sampling_modes must be a down/up dict: {item}")
        unknown = set(modes) - {"down", "up"}
        if unknown:
            raise ValueError(f"lead_sampling_checkpoint_schedule sampling_modes contains unsupported axes: {sorted(unknown)}")
        offload = item.get("offload")
        if offload is not None and not isinstance(offload, dict):
            raise ValueError(f"lead_sampling_checkpoint_schedule offload must be a dict: {item}")
        plans.append(LeadSamplingPlan(first, last, None if down is None else str(down).upper(),
                                      None if up is None else str(up).upper(), modes.get("down"), modes.get("up"),
                                      None if offload is None else dict(offload),
                                      item.get("label", f"lead{first}-{last}:sampling")))
    return sorted(plans, key=lambda p: (p.lead_start, p.lead_end))


def _mode_text(value: str) -> str:
    return value if str(value).lower() == "none" else str(value).upper()


@dataclass
class LeadScheduler:
    """Applies the two schedules to a model before each lead's forward (only when the plan changes) and describes what
    is in force, for the per-lead metrics rows."""

    model: Any
    activation: Dict[str, Any]
    plans: List[LeadPlan] = field(default_factory=list)
    sampling_plans: List[LeadSamplingPlan] = field(default_factory=list)

    def __post_init__(self):
        act = self.activation = self.activation or {}
        self.plans = parse_lead_checkpoint_schedule(act)
        self.sampling_plans = parse_lead_sampling_schedule(act)
        self.base_mode = str(act.get("mode", "torch_recompute"))
        self.base_offload = dict(act.get("offload") or {})
        sampling = act.get("sampling_checkpoint") or {}
        self.base_down, self.base_up = _mode_text(sampling.get("down", "none")), _mode_text(sampling.get("up", "none"))
        modes = act.get("sampling_modes") or {}
        self.base_down_mode = str(modes.get("down", "torch_recompute"))
        self.base_up_mode = str(modes.get("up", "torch_recompute"))
        self._applied_plan = None
        self._applied_layers = None
        self._applied_label = ""
        self._applied_sampling = None
        self._applied_sampling_label = ""

    @property
    def active(self) -> bool:
        return bool(self.plans or self.sampling_plans)

    # ---- look-ups
    def plan_for(self, lead_number: int):
        for p in self.plans:
            if p.covers(lead_number):
                return p.checkpoint_layers, p.activation_mode, p.segment_activation_modes, p.offload, p.label
        return None, self.base_mode, None, self.base_offload, ""

    def sampling_for(self, lead_number: int):
        for p in self.sampling_plans:
            if p.covers(lead_number):
                return (p.down or self.base_down, p.up or self.base_up, p.down_activation_mode or self.base_down_mode,
                        p.up_activation_mode or self.base_up_mode,
                        p.offload if p.offload is not None else self.base_offload, p.label)
        return self.base_down, self.base_up, self.base_down_mode, self.base_up_mode, self.base_offload, ""

    # ---- application
    def _schedulers(self):
        real = self.model.module if hasattr(self.model, "module") else self.model
        return [m.recompute_scheduler for m in real.modules() if getattr(m, "recompute_scheduler", None) is not None]

    def _apply_sampling(self, down, up, down_mode, up_mode, offload) -> int:
        real = self.model.module if hasattr(self.model, "module") else self.model
        touched = 0
        for m in real.modules():
            if not (hasattr(m, "checkpoint_down_mode") or hasattr(m, "checkpoint_up_mode")):
                continue
            cfg = dict(getattr(m, "recompute_config", {}) or {})
            sampling = dict(cfg.get("sampling_checkpoint") or {})
            modes = dict(cfg.get("sampling_modes") or {})
            if down is not None and hasattr(m, "checkpoint_down_mode"):
                m.checkpoint_down_mode = sampling["down"] = cfg["checkpoint_down_mode"] = _mode_text(down)
                modes["down"] = str(down_mode)
            if up is not None and hasattr(m, "checkpoint_up_mode"):
                m.checkpoint_up_mode = sampling["up"] = cfg["checkpoint_up_mode"] = _mode_text(up)
                modes["up"] = str(up_mode)
            cfg.update(sampling_checkpoint=sampling, sampling_modes=modes, offload=dict(offload or {}))
            m.recompute_config = cfg
            for axis in ("down", "up"):
                if hasattr(m, f"{axis}_recompute_config"):
                    sub = dict(activation_config_for_sampling(cfg, axis))
                    sub["offload"] = dict(sub.get("offload") or {}, scope="sampling")
                    setattr(m, f"{axis}_recompute_config", sub)
            touched += 1
        return touched

    def before_lead(self, lead_idx: int) -> None:
        """Install what lead ``lead_idx`` (0-based, as the rollout counts) asks for."""
        number = int(lead_idx) + 1
        if self.sampling_plans:
            down, up, dmode, umode, offload, label = self.sampling_for(number)
            key = (down, up, dmode, umode, json.dumps(offload, sort_keys=True))
            if key != self._applied_sampling:
                if self._apply_sampling(down, up, dmode, umode, offload) <= 0:
                    raise RuntimeError("lead_sampling_checkpoint_schedule is set, but no sampling checkpoint module was found in model")
                self._applied_sampling = key
            if label:
                self._applied_sampling_label = label
        layers, mode, seg, offload, label = self.plan_for(number)
        if layers is not None:
            key = (tuple(map(str, layers)), mode, tuple(seg) if seg is not None else None, json.dumps(offload, sort_keys=True))
            if key != self._applied_plan:
                scheds = self._schedulers()
                if not scheds:
                    raise RuntimeError("lead_checkpoint_schedule is set, but no recompute_scheduler was found in model")
                for s in scheds:
                    s.set_checkpoint_plan(layers, activation_mode=mode, offload_config=offload, segment_activation_modes=seg)
                self._applied_plan, self._applied_layers = key, list(layers)
            self._applied_label = label

    def describe(self, lead_idx: int) -> Dict[str, Any]:
        """The fields of a per-lead metrics row (names as in the reference's ``--memory_timeline_csv``)."""
        number = int(lead_idx) + 1
        layers, mode, seg, offload, label = self.plan_for(number)
        down, up, dmode, umode, _, slabel = self.sampling_for(number)
        return {
            "lead": number,
            "checkpoint_label": label or self._applied_label,
            "checkpoint_layers": json.dumps(layers if layers is not None else self._applied_layers),
            "transformer_activation_mode": mode,
            "transformer_segment_activation_modes": json.dumps(seg if seg is not None else []),
            "transformer_offload": json.dumps(offload, sort_keys=True),
            "sampling_checkpoint_label": slabel or self._applied_sampling_label,
            "sampling_down": down, "sampling_up": up,
            "sampling_down_activation_mode": dmode, "sampling_up_activation_mode": umode,
        }
