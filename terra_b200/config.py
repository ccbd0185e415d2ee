"""YAML model config -> ``(model_archi_params, other_params)``.

Keeps the reference's keys and validation rules (models/model_utils/get_model.py:347-984) and adds the superset
keys this framework needs for other grids and staged head counts:

``height`` / ``width``       grid size (default 2041 x 4320, the GLORYS grid the reference hard-codes)
``depths`` / ``num_heads``   lists: groups of blocks with their head counts (scalar forms stay valid)
``window_size``              scalar or ``[wh, ww]``; the shift is ``(wh // 2, ww // 2)``
``comm_backend``             ``nvlink`` (peer-memory kernels) | ``nccl`` | ``gloo``
"""
from __future__ import annotations

import ast
from typing import Any, Dict, Tuple

import yaml

from .memory.activation import normalize_activation_config
from .parallel.window_assignment import TERRA_M1_ASSIGNMENT_MODES, is_terra_m1_assignment_mode
from .utils.padding import _pair, compute_auto_padded_shape, get_padded_shape

WINDOW_TOPOLOGY_ASSIGNMENT_MODES = {
    "mn": ("regular", "ragged_round_robin"),
    "m1": tuple(sorted(TERRA_M1_ASSIGNMENT_MODES)),
}
SAMPLING_ARCHS = {"credit_hierarchical_swin"}
DEFAULT_HEIGHT, DEFAULT_WIDTH = 2041, 4320


def load_yaml(path: str) -> dict:
    with open(path) as f:
        return yaml.safe_load(f)


def as_tuple2(value, name) -> Tuple[int, int]:
    if isinstance(value, str):
        value = ast.literal_eval(value)
    value = tuple(value)
    if len(value) != 2:
        raise ValueError(f"{name} must have 2 dims, got {value}")
    return int(value[0]), int(value[1])


def get_ranks_per_dp(data_parallel_group_size, world_size):
    return world_size // data_parallel_group_size


def downsample_scale(model_architecture) -> int:
    return 2 if model_architecture in SAMPLING_ARCHS else 1


def build_padding_spec(policy, height, width, patch_size, window_size, model_architecture, padded_shape) -> dict:
    padded_shape = as_tuple2(padded_shape, "padded_shape")
    need, initial, padded_shape = get_padded_shape(height, width, patch_size, window_size, padded_shape=padded_shape)
    ds = downsample_scale(model_architecture)
    if padded_shape[0] % patch_size or padded_shape[1] % patch_size:
        raise ValueError(f"padded_shape={padded_shape} must be divisible by patch_size={patch_size}")
    ph, pw = padded_shape[0] // patch_size, padded_shape[1] // patch_size
    if ph % ds or pw % ds:
        raise ValueError(f"patch token resolution {(ph, pw)} must be divisible by transformer_downsample_scale={ds}")
    th, tw = ph // ds, pw // ds
    wh, ww = _pair(window_size)
    num_windows = (th // wh, tw // ww) if (th % wh == 0 and tw % ww == 0) else None
    return {"policy": policy, "padded_shape": padded_shape, "initial_padding": tuple(initial), "need_padding": bool(need),
            "patch_token_resolution": (ph, pw), "transformer_token_resolution": (th, tw), "num_windows": num_windows,
            "transformer_downsample_scale": ds}


def resolve_padding_spec(model_config, model_architecture, height, width, patch_size, window_size, wp_topo, xfmr_wp_topo,
                         window_assignment_mode) -> dict:
    policy = model_config.get("padding_policy", "scale")
    explicit = model_config.get("padded_shape", model_config.get("resolved_padded_shape"))
    if explicit is not None:
        padded, policy = as_tuple2(explicit, "padded_shape"), "explicit"
    elif policy == "auto":
        padded = compute_auto_padded_shape(height, width, patch_size, window_size, downsample_scale(model_architecture),
                                           wp_topo, xfmr_wp_topo, window_assignment_mode)
    elif policy in ("scale", "legacy", "padding_scale"):
        _, _, padded = get_padded_shape(height, width, patch_size, window_size,
                                        padding_scale=model_config.get("padding_scale", 1))
        policy = "scale"
    else:
        raise ValueError(f"Unsupported padding_policy={policy}")
    return build_padding_spec(policy, height, width, patch_size, window_size, model_architecture, padded)


def validate_window_topology_assignment_pair(window_topology, window_assignment_mode, xfmr_wp_topo):
    if window_topology not in WINDOW_TOPOLOGY_ASSIGNMENT_MODES:
        raise ValueError(f"Unsupported window_topology={window_topology!r}; supported values are: "
                         f"{', '.join(WINDOW_TOPOLOGY_ASSIGNMENT_MODES)}.")
    every = {m for modes in WINDOW_TOPOLOGY_ASSIGNMENT_MODES.values() for m in modes}
    if window_assignment_mode not in every:
        raise ValueError(f"Unsupported window_assignment_mode={window_assignment_mode!r}; supported values are: "
                         f"{', '.join(sorted(every))}.")
    if window_assignment_mode not in WINDOW_TOPOLOGY_ASSIGNMENT_MODES[window_topology]:
        raise ValueError(f"Incompatible window topology configuration: window_topology={window_topology!r} cannot be "
                         f"used with window_assignment_mode={window_assignment_mode!r}.")
    if window_topology == "m1" and xfmr_wp_topo[1] != 1:
        raise ValueError(f"window_topology='m1' requires xfmr_wp_topo=(m, 1), got xfmr_wp_topo={xfmr_wp_topo}.")


def validate_parallel_layout_config(model_architecture, embedding_parallel_type, wp_topo, xfmr_wp_topo, patch_size,
                                    window_size, embedding_dim, num_heads, window_assignment_mode="regular",
                                    window_topology=None, xfmr_sp_size=1, tensor_parallel_size=1, padded_shape=None,
                                    strict_ulysses_heads=False):
    """Divisibility rules of a parallel layout. ``strict_ulysses_heads`` restores the reference's
    ``heads % (sp * tp) == 0`` (its SP shards heads by all-to-all); the K/V-gather SP used here only needs
    ``heads % tp == 0``."""
    if window_topology is None:
        window_topology = "m1" if is_terra_m1_assignment_mode(window_assignment_mode) else "mn"
    validate_window_topology_assignment_pair(window_topology, window_assignment_mode, xfmr_wp_topo)
    sp, tp = int(xfmr_sp_size), int(tensor_parallel_size)
    wp_size = wp_topo[0] * wp_topo[1]
    if wp_size != xfmr_wp_topo[0] * xfmr_wp_topo[1] * sp * tp:
        raise ValueError(f"wp_topo={wp_topo} product must equal xfmr_wp_topo={xfmr_wp_topo} product times "
                         f"xfmr_sp_size={sp} times tensor_parallel_size={tp}")
    if model_architecture in SAMPLING_ARCHS:
        if embedding_parallel_type != "window_linear":
            raise ValueError(f"{model_architecture} uses halo-based sampling blocks, so embedding_parallel_type must be "
                             f"window_linear, got {embedding_parallel_type}")
        if wp_topo[1] != 1:
            raise ValueError(f"{model_architecture} uses halo-based sampling blocks, so data wp_topo must be (m, 1), got {wp_topo}")
    if tuple(wp_topo) != tuple(xfmr_wp_topo):
        if wp_topo[1] != 1:
            raise ValueError(f"layout transform only supports data wp_topo=(m, 1) now, got wp_topo={wp_topo}")
        if embedding_parallel_type != "window_linear":
            raise ValueError(f"layout transform from wp_topo={wp_topo} to xfmr_wp_topo={xfmr_wp_topo} requires window_linear input layout")
    ds = downsample_scale(model_architecture)
    padded_shape = as_tuple2(padded_shape, "padded_shape")
    if padded_shape[0] % patch_size or padded_shape[1] % patch_size:
        raise ValueError(f"padded_shape={padded_shape} must be divisible by patch_size={patch_size}")
    th, tw = padded_shape[0] // patch_size, padded_shape[1] // patch_size
    if th % ds or tw % ds:
        raise ValueError(f"patch token resolution {(th, tw)} must be divisible by transformer_downsample_scale={ds}")
    th, tw = th // ds, tw // ds
    if th % wp_topo[0] or tw % wp_topo[1]:
        raise ValueError(f"transformer token resolution {(th, tw)} must be divisible by data wp_topo={wp_topo}")
    wh, ww = _pair(window_size)
    if th % wh or tw % ww:
        raise ValueError(f"padded token resolution {(th, tw)} must be divisible by window_size={window_size}")
    nh, nw = th // wh, tw // ww
    if nh * nw < xfmr_wp_topo[0] * xfmr_wp_topo[1]:
        raise ValueError(f"too few windows for xfmr_wp_topo={xfmr_wp_topo}: num_windows=({nh}, {nw})")
    if is_terra_m1_assignment_mode(window_assignment_mode) and wp_topo[1] != 1:
        raise ValueError(f"{window_assignment_mode} requires data wp_topo=(m, 1), got wp_topo={wp_topo}")
    if window_assignment_mode == "ragged_round_robin" and tuple(wp_topo) == tuple(xfmr_wp_topo) and wp_topo[1] > 1:
        raise ValueError("ragged_round_robin with data wp_topo == xfmr_wp_topo and n > 1 is not supported. "
                         f"Use data wp_topo=(m, 1), got wp_topo={wp_topo}.")
    if window_assignment_mode == "regular" and (nh % xfmr_wp_topo[0] or nw % xfmr_wp_topo[1]):
        raise ValueError(f"regular xfmr_wp_topo={xfmr_wp_topo} requires num_windows=({nh}, {nw}) to be divisible by the transformer topology")
    if window_assignment_mode == "terra_m1_regular" and nh % xfmr_wp_topo[0]:
        raise ValueError(f"terra_m1_regular xfmr_wp_topo={xfmr_wp_topo} requires num_windows_h={nh} to be divisible by m")
    if window_assignment_mode == "terra_m1_ragged_row" and nh < xfmr_wp_topo[0]:
        raise ValueError(f"terra_m1_ragged_row xfmr_wp_topo={xfmr_wp_topo} requires num_windows_h={nh} >= m")
    if sp > 1 or tp > 1:
        heads = num_heads if isinstance(num_heads, (list, tuple)) else [num_heads]
        div = sp * tp if strict_ulysses_heads else tp
        if embedding_dim % div:
            raise ValueError(f"embedding_dim={embedding_dim} must be divisible by {div}")
        for h in heads:
            if h % div:
                raise ValueError(f"num_heads={h} must be divisible by {div}")
        if (wh * ww) % sp:
            raise ValueError(f"window tokens {wh * ww} must be divisible by xfmr_sp_size={sp}")


def get_model_archi_params_and_other_params(task_type, model_config, data_parallel_group_size=-1, world_size=-1):
    if task_type != "glorys":
        raise ValueError(f"Unsupported task_type: {task_type}. TERRA supports GLORYS only.")
    arch = model_config.get("model_architecture")
    window_size = model_config["window_size"]
    if isinstance(window_size, str):
        window_size = ast.literal_eval(window_size)
    height = int(model_config.get("height", DEFAULT_HEIGHT))
    width = int(model_config.get("width", DEFAULT_WIDTH))
    depths = model_config.get("depths")
    num_heads = model_config["num_heads"]
    num_layers = sum(depths) if depths is not None else model_config["num_layers"]
    archi: Dict[str, Any] = {
        "height": height, "width": width, "num_layers": num_layers, "embedding_dim": model_config["embedding_dim"],
        "num_heads": num_heads, "num_channels": int(model_config.get("num_channels", 93)),
        "patch_size": model_config["patch_size"], "window_size": window_size,
        "padding_scale": model_config.get("padding_scale", 1), "activation": normalize_activation_config(model_config),
        "model_architecture": arch, "depths": depths,
        "use_attn_mask": bool(model_config.get("use_attn_mask", True)),
        "use_relative_position_bias": bool(model_config.get("use_relative_position_bias", True)),
        "USE_FLASH_ATTENTION": bool(model_config.get("USE_FLASH_ATTENTION", model_config.get("use_flash_attention", False))),
    }
    prefetch = str(model_config.get("FSDP_CONFIG7_PREFETCH_POLICY", model_config.get("fsdp_prefetch_policy", "none")) or "none").strip().lower()
    if prefetch not in ("overlap", "conservative", "none"):
        raise ValueError(f"FSDP_CONFIG7_PREFETCH_POLICY/fsdp_prefetch_policy must be one of 'overlap', 'conservative', or 'none', got {prefetch!r}")
    archi["FSDP_CONFIG7_PREFETCH_POLICY"] = prefetch
    sampling_cfg = int(model_config.get("FSDP_SAMPLING_WRAPPER_CFG", model_config.get("fsdp_sampling_wrapper_cfg", 0)))
    if sampling_cfg not in (0, 1, 2):
        raise ValueError("FSDP_SAMPLING_WRAPPER_CFG/fsdp_sampling_wrapper_cfg must be one of 0, 1, or 2")
    archi["FSDP_SAMPLING_WRAPPER_CFG"] = sampling_cfg

    other: Dict[str, Any] = {}
    model_type = model_config["model_type"]
    if model_type == "sequential":
        other.update(mp_size=1, wp_topo=(1, 1), xfmr_wp_topo=(1, 1), xfmr_sp_size=1, tensor_parallel_size=1,
                     domain_topo=(1, 1), sp_tp_placement="tp_first", embedding_parallel_type=None,
                     attn_parallel_type=None, mlp_parallel_type=None, window_assignment_mode="regular",
                     window_topology="mn")
    elif model_type == "parallel":
        ranks_per_dp = get_ranks_per_dp(data_parallel_group_size, world_size)
        if ranks_per_dp <= 0:
            raise ValueError(f"ranks_per_dp must be positive for window parallel, got {ranks_per_dp}")
        sp = int(model_config.get("xfmr_sp_size", 1))
        tp = int(model_config.get("tensor_parallel_size", 1))
        mode = model_config.get("window_assignment_mode", "regular")
        topology = model_config.get("window_topology", "m1" if is_terra_m1_assignment_mode(mode) else "mn")
        placement = model_config.get("sp_tp_placement", model_config.get("topology_placement", "tp_first"))
        ept = model_config.get("embedding_parallel_type", "window_linear")
        if ept not in ("window_embedding", "domain_parallel", "window_domain", "window_linear"):
            raise ValueError(f"unsupported embedding_parallel_type {ept}")
        wp_topo = model_config.get("wp_topo")
        if wp_topo is None:
            wp_topo = (ranks_per_dp, 1)
        else:
            wp_topo = as_tuple2(wp_topo, "wp_topo")
            if wp_topo[0] * wp_topo[1] != ranks_per_dp:
                raise ValueError(f"wp_topo product {wp_topo} must equal ranks_per_dp={ranks_per_dp}")
        xfmr = model_config.get("xfmr_wp_topo")
        if xfmr is None:
            xfmr = wp_topo
        else:
            xfmr = as_tuple2(xfmr, "xfmr_wp_topo")
            if xfmr[0] * xfmr[1] * sp * tp != wp_topo[0] * wp_topo[1]:
                raise ValueError(f"xfmr_wp_topo product {xfmr} times xfmr_sp_size={sp} times tensor_parallel_size={tp} "
                                 f"must equal wp_topo product {wp_topo}")
        spec = resolve_padding_spec(model_config, arch, height, width, archi["patch_size"], window_size, wp_topo, xfmr, mode)
        archi.update(padding_spec=spec, padded_shape=spec["padded_shape"], initial_padding=spec["initial_padding"],
                     padding_policy=spec["policy"])
        validate_parallel_layout_config(arch, ept, wp_topo, xfmr, archi["patch_size"], window_size, archi["embedding_dim"],
                                        num_heads, mode, topology, sp, tp, spec["padded_shape"],
                                        strict_ulysses_heads=bool(model_config.get("strict_ulysses_heads", False)))
        other.update(mp_size=1, wp_topo=wp_topo, xfmr_wp_topo=xfmr, xfmr_sp_size=sp, tensor_parallel_size=tp,
                     sp_tp_placement=placement, domain_topo=(1, 1), embedding_parallel_type=ept, attn_parallel_type="wp",
                     mlp_parallel_type="wp", window_assignment_mode=mode, window_topology=topology)
    else:
        raise ValueError(f"unrecognized model_type {model_type}")

    if "padding_spec" not in archi:
        spec = resolve_padding_spec(model_config, arch, height, width, archi["patch_size"], window_size, other["wp_topo"],
                                    other["xfmr_wp_topo"], other["window_assignment_mode"])
        archi.update(padding_spec=spec, padded_shape=spec["padded_shape"], initial_padding=spec["initial_padding"],
                     padding_policy=spec["policy"])
    other["padding_spec"] = archi["padding_spec"]
    other["use_splited_data"] = True
    other["norm_type"] = model_config.get("norm_type", "zs")
    other["data_precision"] = model_config.get("data_precision", "fp16")
    other["comm_backend"] = model_config.get("comm_backend", "nvlink")
    root = model_config.get("glorys_data_root") or model_config.get("sequential_data_root") or model_config.get("data_root")
    if root is not None:
        other["glorys_data_root"] = root
    return archi, other
