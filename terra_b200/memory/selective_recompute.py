"""Turns an activation config into non-overlapping ``[start, end)`` transformer-block segments.

Same observable behaviour as the reference scheduler (core/checkpoint/selective_recompute.py:8-209):
``execution_segments()`` yields ``(start, end, checkpoint?)`` covering every block once, plans can be replaced
between rollout leads with ``set_checkpoint_plan``.
"""
from __future__ import annotations

from typing import Dict, Iterable, Iterator, List, Optional, Sequence, Tuple

from .activation import (activation_config_for_layer, normalize_activation_config, normalize_activation_mode,
                         parse_layer_entry)

_SAMPLING_TOKENS = {"d0", "d1", "d2", "u0", "u1", "u2"}


class SelectiveRecomputeScheduler:
    def __init__(self, config=None, depth=0, input_resolution=None, hidden_dim=None, module_name="transformer"):
        self.depth = int(depth)
        self.input_resolution = input_resolution
        self.hidden_dim = hidden_dim
        self.module_name = module_name
        self._install(normalize_activation_config(config=config))

    # ------------------------------------------------------------------ configuration
    def _install(self, config: dict) -> None:
        self.config = config
        self.enabled = bool(config.get("enabled", False))
        self.mode = self.impl = config.get("mode", "none")
        self.policy = str(config.get("policy", "none")).strip().lower()
        self.checkpoint_every_n_layers = int(config.get("checkpoint_every_n_layers", 4))
        self._rebuild()

    def _rebuild(self) -> None:
        self.checkpoint_segments = self._plan()
        self.block_indices = {i for s, e in self.checkpoint_segments for i in range(s, e)}

    def set_checkpoint_layers(self, checkpoint_layers) -> None:
        self._replan(checkpoint_layers)

    def set_checkpoint_plan(self, checkpoint_layers, activation_mode=None, offload_config=None,
                            segment_activation_modes=None) -> None:
        """Replace the plan between rollout leads: new layer entries and, optionally, a new default mode, offload
        options and one mode per entry."""
        changes = {}
        if activation_mode is not None:
            changes["mode"] = str(activation_mode)
        if offload_config is not None:
            changes["offload"] = dict(offload_config)
        if segment_activation_modes is not None:
            changes["layer_modes"] = self._modes_by_first_block(checkpoint_layers, segment_activation_modes)
        self._replan(checkpoint_layers, changes)

    def _modes_by_first_block(self, entries, modes) -> Dict[int, str]:
        """``{first block of segment i: mode i}`` - the form in which per-layer modes are stored."""
        firsts = [start for start, _ in self._from_entries(list(entries))]
        modes = list(modes)
        if len(modes) != len(firsts):
            raise ValueError(f"segment_activation_modes must match checkpoint_layers: {len(modes)} != {len(firsts)}")
        return {int(b): normalize_activation_mode(m) for b, m in zip(firsts, modes)}

    def _replan(self, checkpoint_layers, changes: Optional[dict] = None) -> None:
        raw = {k: v for k, v in self.config.items() if k != "checkpoint_segments"}
        raw["checkpoint_layers"] = list(checkpoint_layers) if changes is not None else checkpoint_layers
        if changes:
            raw.update(changes)
            raw = normalize_activation_config(config=raw)
            # the normaliser derives segments from the layer entries; the plan below is built from the entries themselves
            raw["checkpoint_layers"] = checkpoint_layers
            raw.pop("checkpoint_segments", None)
            self.enabled = bool(raw.get("enabled", False))
            self.mode = self.impl = raw.get("mode", "none")
        self.config = raw
        self._rebuild()

    # ------------------------------------------------------------------ planning
    def _sanitise(self, segments: Iterable[Tuple[int, int]]) -> List[Tuple[int, int]]:
        out, last_end = [], -1
        for start, end in segments:
            start = min(max(int(start), 0), self.depth)
            end = min(max(int(end), 0), self.depth)
            if end <= start:
                continue
            if start < last_end:
                raise ValueError("activation checkpoint segments must be non-overlapping and sorted, "
                                 f"but got segment ({start}, {end}) after previous end {last_end}")
            out.append((start, end))
            last_end = end
        return out

    def _from_entries(self, entries) -> List[Tuple[int, int]]:
        segs = []
        for entry in entries:
            if not isinstance(entry, int) and str(entry).strip().lower() in _SAMPLING_TOKENS:
                continue
            segs.append(parse_layer_entry(entry))
        return self._sanitise(segs)

    def _singletons(self, indices) -> List[Tuple[int, int]]:
        return self._sanitise((i, i + 1) for i in sorted(set(indices)))

    def _plan(self) -> List[Tuple[int, int]]:
        if not self.enabled or self.policy == "none":
            return []
        if self.policy == "larger_wrapper":
            return self._sanitise(self.config.get("checkpoint_segments", []))
        explicit = self.config.get("checkpoint_layers")
        if explicit is None:
            explicit = self.config.get("block_indices")
        if explicit is not None:
            return self._from_entries(explicit)
        if self.policy == "full_checkpoint" or bool(self.config.get("full_checkpoint", False)):
            return self._singletons(range(self.depth))
        if self.policy == "uniform":
            n = max(1, self.checkpoint_every_n_layers)
            return self._singletons(i for i in range(self.depth) if i % n == 0)
        raise ValueError(f"Unsupported recompute policy: {self.policy}")

    # ------------------------------------------------------------------ queries
    def should_checkpoint(self, block_idx) -> bool:
        return self.enabled and int(block_idx) in self.block_indices

    def config_for_block(self, block_idx) -> dict:
        return activation_config_for_layer(self.config, block_idx)

    def execution_segments(self) -> Iterator[Tuple[int, int, bool]]:
        ends = dict(self.checkpoint_segments) if self.enabled else {}
        i = 0
        while i < self.depth:
            if i in ends:
                yield i, ends[i], True
                i = ends[i]
            else:
                yield i, i + 1, False
                i += 1

    def summary(self) -> dict:
        cfg = self.config
        plan = {"block_indices": sorted(self.block_indices),
                "checkpoint_segments": [list(seg) for seg in self.checkpoint_segments],
                "segment_activation_modes": [self.config_for_block(first)["mode"] for first, _ in self.checkpoint_segments],
                "layer_modes": dict(sorted(cfg.get("layer_modes", {}).items()))}
        sampling = {"sampling_checkpoint": dict(cfg.get("sampling_checkpoint", {"down": "none", "up": "none"})),
                    "sampling_modes": dict(cfg.get("sampling_modes", {}))}
        shape = {name: getattr(self, name) for name in ("enabled", "mode", "policy", "depth", "input_resolution", "hidden_dim")}
        return {**shape, **plan, **sampling}
