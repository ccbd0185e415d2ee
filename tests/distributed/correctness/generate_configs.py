#!/usr/bin/env python3
"""Writes the YAML files of the serial-versus-parallel convergence experiment (reference:
tests/distributed/correctness/generate_configs.py). Five cases share model, data and optimiser settings and differ
only in the layout: a serial baseline and four factorizations of 8 model-parallel ranks,
WP 8, WP 4 x SP 2, WP 4 x TP 2 and WP 2 x SP 2 x TP 2, each replicated ``DATA_PARALLEL_SIZE`` times.

Everything is parameterised by environment variables (see ``env.sh``) so that the same generator serves the
16-GPU experiment, an 8-GPU node (``MODEL_PARALLEL_SIZE=8 DATA_PARALLEL_SIZE=1``) and a tiny CPU rehearsal
(``MODEL_PARALLEL_SIZE=2`` with small shapes)."""
from __future__ import annotations

import os
from dataclasses import dataclass
from pathlib import Path

import yaml

HERE = Path(__file__).resolve().parent


def _env(name, default, cast=str):
    return cast(os.environ.get(name, default))


@dataclass(frozen=True)
class Case:
    name: str
    label: str
    wp: int      # window-parallel groups of the Swin stage (0 = serial model)
    sp: int
    tp: int
    optimizer_config: int


def cases(mp: int):
    """The case list for ``mp`` model-parallel ranks (``mp`` a multiple of 4 for the full set)."""
    out = [Case("seq_fsdp", "Serial", 0, 1, 1, _env("SEQ_OPTIMIZER_CONFIG", 7, int)),
           Case("topo_wp", "TERRA WP", mp, 1, 1, 7)]
    if mp % 2 == 0:
        out.append(Case("topo_wp_sp", "TERRA WP+SP", mp // 2, 2, 1, 7))
        out.append(Case("topo_wp_tp", "TERRA WP+TP", mp // 2, 1, 2, 9))
    if mp % 4 == 0:
        out.append(Case("topo_wp_sp_tp", "TERRA WP+SP+TP", mp // 4, 2, 2, 9))
    return out


def build(case: Case, mp: int) -> dict:
    layers = _env("SMALL_NUM_LAYERS", 10, int)
    dp = _env("DATA_PARALLEL_SIZE", 2, int)
    cfg = {
        "description": f"correctness_{case.name}",
        "experiment_name": "seq_ddp_vs_parallel_correctness",
        "case_name": case.name,
        "case_label": case.label,
        "topology_label": "Serial" if case.wp == 0 else f"Topo({case.wp},1,{case.sp},{case.tp})",
        "global_gpu_count": mp * dp,
        "data_parallel_size": dp,
        "train_path": f"./tests/distributed/correctness/train_runs/{case.name}",
        "saved_data_path": f"./tests/distributed/correctness/saved_data/{case.name}",
        "ckpt_start": False, "ckpt_epoch": 0, "load_saved_data_dict": False, "clip_grad": False,
        "use_fake_input": _env("USE_FAKE_INPUT", 0, int) == 1,
        "task_type": "glorys",
        "model_architecture": _env("MODEL_ARCHITECTURE", "credit_hierarchical_swin"),
        "num_channels": _env("NUM_CHANNELS", 93, int),
        "optimizer_config": case.optimizer_config,
        "fsdp_checkpoint_type": "full",
        "precision": _env("PRECISION", "bf16"),
        "half_model": False,
        "use_splited_data": False,
        "norm_type": "mm",
        "model_type": "sequential" if case.wp == 0 else "parallel",
        "micro_batch_size": _env("MICRO_BATCH_SIZE", 1, int),
        "num_workers": _env("NUM_WORKERS", 2, int),
        "learning_rate": _env("LEARNING_RATE", 1e-4, float),
        "warmup_steps": _env("WARMUP_STEPS", 10, int),
        "loss_func": _env("LOSS_FUNC", "L1"),
        "padding_policy": "explicit",
        "padded_shape": [_env("PADDED_SHAPE_H", 2304, int), _env("PADDED_SHAPE_W", 4352, int)],
        "padding_scale": _env("PADDING_SCALE", 2, int),
        "patch_size": _env("PATCH_SIZE", 4, int),
        "window_size": _env("WINDOW_SIZE", 8, int),
        "num_layers": layers,
        "embedding_dim": _env("SMALL_EMBEDDING_DIM", 1024, int),
        "num_heads": _env("SMALL_NUM_HEADS", 8, int),
        "kaiming_init": True,
        "use_attn_mask": True,
        "use_relative_position_bias": True,
        "activation": {
            "mode": _env("ACTIVATION_MODE", "torch_recompute"),
            "policy": _env("ACTIVATION_POLICY", "uniform"),
            "checkpoint_layers": list(range(layers)),
            "sampling_checkpoint": {"down": _env("SAMPLING_CHECKPOINT_DOWN", "D1"), "up": _env("SAMPLING_CHECKPOINT_UP", "U1")},
        },
    }
    if "HEIGHT" in os.environ:
        cfg["height"], cfg["width"] = _env("HEIGHT", 0, int), _env("WIDTH", 0, int)
    if case.wp:
        if case.wp * case.sp * case.tp != mp:
            raise ValueError(f"{case.name}: WP*SP*TP = {case.wp}*{case.sp}*{case.tp} != {mp}")
        cfg.update({
            "embedding_parallel_type": "window_linear",
            "wp_topo": f"({mp}, 1)",
            "xfmr_wp_topo": f"({case.wp}, 1)",
            "xfmr_sp_size": case.sp,
            "tensor_parallel_size": case.tp,
            "sp_tp_placement": "tp_first",
            "window_assignment_mode": _env("WINDOW_ASSIGNMENT_MODE", "terra_m1_ragged_auto"),
        })
    return cfg


def main():
    mp = _env("MODEL_PARALLEL_SIZE", 8, int)
    out_dir = Path(_env("CONFIG_DIR", str(HERE / "configs")))
    out_dir.mkdir(parents=True, exist_ok=True)
    wanted = set(_env("CASES", "").split()) or None
    for case in cases(mp):
        if wanted and case.name not in wanted:
            continue
        path = out_dir / f"correctness_{case.name}.yaml"
        path.write_text(yaml.safe_dump(build(case, mp), sort_keys=False))
        print(path)


if __name__ == "__main__":
    main()
