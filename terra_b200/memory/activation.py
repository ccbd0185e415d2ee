"""Parsing of the ``activation:`` YAML block and dispatch of one checkpointed call.

Semantics follow the reference parser (core/checkpoint/activation.py:24-319): three modes with aliases,
policies ``full_checkpoint`` / ``uniform`` / ``larger_wrapper`` / explicit ``checkpoint_layers``,
``sampling_checkpoint.{down,up}``, per-layer ``layer_modes``, per-axis ``sampling_modes``, the legacy
``selective_recompute:`` block as an input alias, and a hard error for the retired sampling keys.
"""
from __future__ import annotations

import copy
from typing import Any, Dict, Iterable, List, Optional, Tuple

NONE, RECOMPUTE, OFFLOAD = "none", "torch_recompute", "cpu_boundary_offload_recompute"

_MODE_TABLE = {
    NONE: ("none", "no", "off", "disabled"),
    RECOMPUTE: ("torch", "torch_checkpoint", "torch_recompute"),
    OFFLOAD: ("boundary_offload", "cpu_boundary_offload", "cpu_boundary_offload_recompute", "cpu_offload_boundary"),
}
_MODE_LOOKUP = {alias: canon for canon, aliases in _MODE_TABLE.items() for alias in aliases}

_SAMPLING_TABLE = {
    "down": {"D0": ("d0", "fused", "patch_embed_down", "patch_sampling"), "D1": ("d1", "split", "granular")},
    "up": {"U0": ("u0", "fused", "up_patch_recovery", "patch_sampling"), "U1": ("u1", "split", "granular")},
}
_SAMPLING_OFF = ("", "none", "no", "off", "false", "0", "disabled")
_RETIRED_KEYS = ("checkpoint_sampling_blocks", "checkpoint_patch_sampling_blocks", "checkpoint_patch_blocks",
                 "checkpoint_patch_embed_down", "checkpoint_up_patch_recovery")


def normalize_activation_mode(mode) -> str:
    if mode is None:
        return NONE
    key = str(mode).strip().lower()
    try:
        return _MODE_LOOKUP[key]
    except KeyError:
        raise ValueError(f"Unsupported activation mode: {mode}") from None


def normalize_sampling_mode(value, axis: str) -> str:
    if value is None or str(value).strip().lower() in _SAMPLING_OFF:
        return "none"
    key = str(value).strip().lower()
    for canon, aliases in _SAMPLING_TABLE[axis].items():
        if key in aliases:
            return canon
    valid = ", ".join(["none"] + sorted(_SAMPLING_TABLE[axis]))
    raise ValueError(f"Unsupported {axis} sampling checkpoint mode: {value}. Valid modes: {valid}")


def parse_layer_entry(entry) -> Tuple[int, int]:
    """``3`` -> (3, 4); ``'2-5'`` -> (2, 6) (inclusive range)."""
    if isinstance(entry, int):
        return entry, entry + 1
    text = str(entry).strip()
    if not text:
        raise ValueError("Empty activation checkpoint layer entry")
    if text.lstrip("+-").isdigit():
        return int(text), int(text) + 1
    if "-" not in text:
        raise ValueError(f"Unsupported activation checkpoint layer entry: {entry}")
    lo, hi = (part.strip() for part in text.split("-", 1))
    if not lo or not hi:
        raise ValueError(f"Malformed activation checkpoint layer range: {entry}")
    lo, hi = int(lo), int(hi)
    if hi < lo:
        raise ValueError(f"Invalid activation checkpoint layer range: {entry}")
    return lo, hi + 1


def _listify(value) -> List[Any]:
    if value is None:
        return []
    return list(value) if isinstance(value, (list, tuple, set)) else [value]


def _layer_modes(raw) -> Dict[int, str]:
    """Accepts ``{layer: mode}`` or ``{mode: [layers]}``."""
    if raw is None:
        return {}
    if not isinstance(raw, dict):
        raise ValueError("activation.layer_modes must be a dict")
    out: Dict[int, str] = {}
    for key, value in raw.items():
        text = str(key).strip()
        if text.lstrip("+-").isdigit():
            out[int(text)] = normalize_activation_mode(value)
        else:
            mode = normalize_activation_mode(text)
            for idx in _listify(value):
                out[int(idx)] = mode
    return out


def _sampling_strategy_modes(raw) -> Dict[str, str]:
    if raw is None:
        return {}
    if not isinstance(raw, dict):
        raise ValueError("activation.sampling_modes must be a dict with optional down/up fields")
    out = {}
    for key, value in raw.items():
        axis = str(key).strip().lower()
        if axis not in ("down", "up"):
            raise ValueError(f"Unsupported activation.sampling_modes key: {key}. Expected down/up")
        out[axis] = normalize_activation_mode(value)
    return out


def normalize_activation_config(model_config: Optional[dict] = None, config=None) -> dict:
    """Canonical dict with keys mode/enabled/policy/checkpoint_layers/checkpoint_segments/
    checkpoint_down_mode/checkpoint_up_mode/sampling_checkpoint/layer_modes/sampling_modes/offload."""
    if config is not None:
        raw = copy.deepcopy(config)
    elif model_config is not None and model_config.get("activation") is not None:
        raw = copy.deepcopy(model_config["activation"])
    elif model_config is not None and model_config.get("selective_recompute") is not None:
        raw = copy.deepcopy(model_config["selective_recompute"])
        legacy_on = bool(raw.get("enabled", False))
        raw["mode"] = normalize_activation_mode(raw.get("backend", raw.get("impl", "torch"))) if legacy_on else NONE
    else:
        raw = {"mode": NONE}
    if isinstance(raw, str):
        raw = {"mode": raw}

    mode = raw.get("mode")
    if mode is None:
        mode = NONE if raw.get("enabled") is False else raw.get("backend", raw.get("impl", NONE))
    mode = normalize_activation_mode(mode)
    out = dict(raw)
    out["mode"] = mode
    out["enabled"] = mode != NONE
    if not out["enabled"]:
        out.update(policy="none", checkpoint_layers=[], block_indices=[], checkpoint_segments=[],
                   checkpoint_patch_embed=False, checkpoint_patch_recovery=False, checkpoint_down_mode="none",
                   checkpoint_up_mode="none", sampling_checkpoint={"down": "none", "up": "none"})
        return out

    out["policy"] = out.get("policy") or "full_checkpoint"
    if out.get("checkpoint_layers") is None and out.get("block_indices") is not None:
        out["checkpoint_layers"] = out["block_indices"]

    retired = [k for k in _RETIRED_KEYS if k in out]
    if retired:
        raise ValueError(f"Deprecated activation sampling config key(s): {', '.join(retired)}. "
                         "Use activation.sampling_checkpoint.down/up instead.")
    sampling = out.get("sampling_checkpoint")
    if sampling is None:
        down, up = "none", "none"
    elif isinstance(sampling, dict):
        down = normalize_sampling_mode(sampling.get("down"), "down")
        up = normalize_sampling_mode(sampling.get("up"), "up")
    else:
        raise ValueError("activation.sampling_checkpoint must be a dict with optional down/up fields")

    segments: List[Tuple[int, int]] = []
    if str(out["policy"]).strip().lower() == "larger_wrapper":
        for item in _listify(out.get("checkpoint_layers")):
            token = str(item).strip().lower()
            if token in ("d0", "d1"):
                down = normalize_sampling_mode(token, "down")
            elif token in ("u0", "u1"):
                up = normalize_sampling_mode(token, "up")
            else:
                segments.append(parse_layer_entry(item))
    out["checkpoint_segments"] = segments
    out["checkpoint_down_mode"], out["checkpoint_up_mode"] = down, up
    out["sampling_checkpoint"] = {"down": down, "up": up}
    out["layer_modes"] = _layer_modes(out.get("layer_modes"))
    out["sampling_modes"] = _sampling_strategy_modes(out.get("sampling_modes"))
    out["checkpoint_patch_embed"] = bool(out.get("checkpoint_patch_embed", False))
    out["checkpoint_patch_recovery"] = bool(out.get("checkpoint_patch_recovery", False))
    return out


def activation_config_with_mode(config, mode) -> dict:
    out = dict(normalize_activation_config(config=config))
    out["mode"] = normalize_activation_mode(mode)
    out["enabled"] = out["mode"] != NONE
    return out


def activation_config_for_layer(config, layer_idx: int) -> dict:
    base = normalize_activation_config(config=config)
    override = base.get("layer_modes", {}).get(int(layer_idx))
    return base if override is None else activation_config_with_mode(base, override)


def activation_config_for_sampling(config, axis: str) -> dict:
    base = normalize_activation_config(config=config)
    override = base.get("sampling_modes", {}).get(str(axis).strip().lower())
    return base if override is None else activation_config_with_mode(base, override)


def activation_checkpoint(function, *args, activation_config=None, mode=None):
    """Run ``function(*args)`` plainly, under recompute, or under recompute with its inputs parked in pinned
    host memory until backward needs them."""
    cfg = normalize_activation_config(config=activation_config if activation_config is not None else {"mode": mode})
    if cfg["mode"] == NONE:
        return function(*args)
    if cfg["mode"] == RECOMPUTE:
        from torch.utils.checkpoint import checkpoint

        return checkpoint(function, *args, use_reentrant=False, preserve_rng_state=True)
    if cfg["mode"] == OFFLOAD:
        from .boundary_offload import checkpoint as offload_checkpoint

        return offload_checkpoint(function, *args, offload_config=cfg.get("offload"))
    raise ValueError(f"Unsupported activation mode: {cfg['mode']}")
