"""Metric files of the test harnesses, in the reference's column and key names.

The pretraining harness writes one CSV row per step and a JSON record of the run
(reference: train_scripts/test_pretrain.py:515-664); the rollout harness the same with its own columns
(reference: train_scripts/test_finetune.py:1085-1206). Analysis scripts written against the reference's files read
these unchanged; columns that only this framework records (``forward_time_s`` in the pretraining rows, the offload
counters in the rollout rows) come after the reference's.

``gather_run_facts`` holds the collectives, so every rank calls it; the writers run on the logging rank only.
"""
from __future__ import annotations

import csv
import json
import os
from typing import Dict, List, Optional, Sequence

import torch.distributed as dist

from terra_b200.checkpoint_io import FSDP_OPTIMIZER_CONFIGS

PRETRAIN_COLUMNS = (
    "iter", "loss", "output_sum", "output_dtype", "peak_memory_mb", "step_time_s", "padding_policy", "padding_scale",
    "input_shape", "need_padding", "padded_shape", "initial_padding", "padding_overhead_pct", "patch_token_resolution",
    "transformer_token_resolution", "num_windows", "transformer_downsample_scale",
)
FINETUNE_COLUMNS = (
    "iter", "lead_time", "loss_reduction", "loss", "loss_per_lead", "loss_sum_estimated", "output_sum", "output_dtype",
    "peak_memory_mb", "step_time_s", "forward_time_s", "rest_time_s", "flops_tflops", "load_data_time_s",
)
LEAD_COLUMNS = (
    "iter", "lead", "checkpoint_label", "checkpoint_layers", "transformer_activation_mode",
    "transformer_segment_activation_modes", "transformer_offload", "sampling_checkpoint_label", "sampling_down",
    "sampling_up", "sampling_down_activation_mode", "sampling_up_activation_mode", "allocated_memory_mb",
    "reserved_memory_mb", "peak_memory_mb", "loss",
)


def _plain(v):
    """Tuples of ints print like the reference's (``str`` of a tuple) whether the config held a list or a tuple."""
    if isinstance(v, (list, tuple)):
        return tuple(_plain(x) for x in v)
    return v


def padding_facts(archi: dict) -> Dict[str, object]:
    """The padding decision of the run: policy, shapes before and after, the overhead and the token grids."""
    spec = archi.get("padding_spec", {}) or {}
    padded = archi.get("padded_shape", spec.get("padded_shape"))
    shape = (archi.get("height"), archi.get("width"))
    overhead = None
    if padded is not None and None not in shape:
        overhead = (int(padded[0]) * int(padded[1]) / (int(shape[0]) * int(shape[1])) - 1.0) * 100.0
    return {
        "padding_policy": archi.get("padding_policy", spec.get("policy")),
        "padding_scale": archi.get("padding_scale"),
        "input_shape": shape,
        "need_padding": spec.get("need_padding"),
        "padded_shape": _plain(padded),
        "initial_padding": _plain(archi.get("initial_padding", spec.get("initial_padding"))),
        "padding_overhead_pct": overhead,
        "patch_token_resolution": _plain(spec.get("patch_token_resolution")),
        "transformer_token_resolution": _plain(spec.get("transformer_token_resolution")),
        "num_windows": _plain(spec.get("num_windows")),
        "transformer_downsample_scale": spec.get("transformer_downsample_scale"),
    }


def _gather(value, kind=float) -> List:
    """One scalar from every rank, in rank order (the value itself without a process group)."""
    if not (dist.is_available() and dist.is_initialized()):
        return [kind(value)]
    out = [None] * dist.get_world_size()
    dist.all_gather_object(out, kind(value))
    return out


def gather_run_facts(session, rows: Sequence[dict], offload_stats: Optional[dict] = None) -> Dict[str, object]:
    """Per-rank parameter counts, last-step peak memory and step time, and the offload counters. Collective."""
    whole = sum(p.numel() for p in session.model.parameters())
    sharder = getattr(session.model, "_param_sharder", None)
    # with sharded parameters a rank holds its owned slices (alignment padding included); otherwise the whole model
    local = int(sharder.owned_numel()) if sharder is not None else whole
    pre_wrap = int(getattr(session.model, "pre_wrap_parameter_count", whole))
    by_rank = _gather(local, int)
    pre_by_rank = _gather(pre_wrap, int)
    tp = int(session.other.get("tensor_parallel_size", 1))
    sharded_state = sharder is not None or session.cfg.get("optimizer_config") in FSDP_OPTIMIZER_CONFIGS
    if sharder is not None:
        total, method = max(pre_by_rank), "pre_wrap_full_count_before_fsdp_wrap"
    elif tp > 1:
        total, method = None, "tp_sharded_local_count_only"
    else:
        total, method = max(pre_by_rank), "pre_wrap_replicated_full_count"
    facts = {
        "parameter_count": {
            "local_parameter_count": local, "pre_wrap_parameter_count": pre_wrap,
            "post_wrap_local_parameter_counts_by_rank": by_rank, "pre_wrap_parameter_counts_by_rank": pre_by_rank,
            "global_parameter_count": total, "parameter_count_method": method,
            "fsdp_group_size": session.world if sharded_state else 1, "tensor_parallel_size": tp,
        },
        "peak_memory_last_by_rank": _gather(rows[-1]["peak_memory_mb"]) if rows else [],
        "step_time_last_by_rank": _gather(rows[-1]["step_time_s"]) if rows else [],
    }
    if offload_stats is not None:
        if dist.is_available() and dist.is_initialized():
            stats = [None] * dist.get_world_size()
            dist.all_gather_object(stats, dict(offload_stats))
        else:
            stats = [dict(offload_stats)]
        facts["boundary_offload_stats_by_rank"] = stats
    return facts


def _run_metadata(session, args, steps: int) -> Dict[str, object]:
    c, o = session.cfg, session.other
    return {
        "model_cfg": os.path.abspath(args.model_cfg),
        "steps": steps,
        "world_size": session.world,
        "data_parallel_group_size": session.dp,
        "ranks_per_dp": session.world // max(1, session.dp),
        "task_type": session.task_type,
        "model_architecture": c.get("model_architecture"),
        "model_type": session.model_type,
        "optimizer_config": c.get("optimizer_config"),
        "precision": c.get("precision"),
        "micro_batch_size": c.get("micro_batch_size"),
        "learning_rate": c.get("learning_rate"),
        "wp_topo": _plain(o.get("wp_topo")),
        "xfmr_wp_topo": _plain(o.get("xfmr_wp_topo")),
        "xfmr_sp_size": o.get("xfmr_sp_size", 1),
        "tensor_parallel_size": o.get("tensor_parallel_size", 1),
        "sp_tp_placement": o.get("sp_tp_placement"),
        "window_assignment_mode": o.get("window_assignment_mode", "regular"),
        "num_layers": c.get("num_layers"),
        "embedding_dim": c.get("embedding_dim"),
        "num_heads": c.get("num_heads"),
        "patch_size": c.get("patch_size"),
        "window_size": c.get("window_size"),
    }


def _write_csv(path: str, columns: Sequence[str], rows: Sequence[dict]) -> None:
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    extra = [k for k in dict.fromkeys(k for r in rows for k in r) if k not in columns]
    with open(path, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=list(columns) + extra, extrasaction="ignore")
        w.writeheader()
        w.writerows(rows)


def _write_json(path: str, record: dict) -> None:
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        json.dump(record, f, indent=2, default=str)


def json_path_for(args) -> Optional[str]:
    """``--metrics_json`` if given, else the CSV's name with ``.json``; nothing with ``--metrics_no_json``."""
    if getattr(args, "metrics_no_json", False):
        return None
    if args.metrics_json:
        return os.path.abspath(args.metrics_json)
    if args.metrics_csv:
        return os.path.splitext(os.path.abspath(args.metrics_csv))[0] + ".json"
    return None


def write_pretrain_metrics(session, args, rows: Sequence[dict], facts: dict, flops, extra: Optional[dict] = None):
    """``rows``: dicts with iter, loss, output_sum, output_dtype, peak_memory_mb, step_time_s (and this framework's
    ``forward_time_s``). ``flops``: a ``FlopsSummary``. ``extra``: further keys for the JSON record."""
    pad = padding_facts(session.archi)
    csv_path = os.path.abspath(args.metrics_csv) if args.metrics_csv else None
    if csv_path:
        text = {k: (str(v) if isinstance(v, tuple) else v) for k, v in pad.items()}
        _write_csv(csv_path, PRETRAIN_COLUMNS, [dict(r, **text) for r in rows])
        print(f"[test_pretrain] wrote metrics csv to {csv_path}")
    json_path = json_path_for(args)
    if json_path is None:
        return
    counts = facts["parameter_count"]
    record = _run_metadata(session, args, len(rows))
    record.update(pad)
    record["padding_scale"] = session.cfg.get("padding_scale")
    record["metrics_csv"] = csv_path
    record["parameter_count"] = counts
    for k in ("local_parameter_count", "pre_wrap_parameter_count", "global_parameter_count", "parameter_count_method",
              "post_wrap_local_parameter_counts_by_rank", "pre_wrap_parameter_counts_by_rank", "fsdp_group_size"):
        record[k] = counts[k]
    record.update(flops.as_metadata())
    record.update(extra or {})
    _write_json(json_path, record)
    print(f"[test_pretrain] wrote metrics json to {json_path}")


def finetune_row(i: int, lead: int, reduction: str, loss: float, output_sum: float, output_dtype, peak: float,
                 step_time: float, forward_time: Optional[float], load_time: Optional[float],
                 local_flops_per_step: float = 0.0, **more) -> dict:
    """One rollout step in the reference's columns; ``more`` holds this framework's additional columns."""
    n = max(1, lead)
    row = {
        "iter": i, "lead_time": lead, "loss_reduction": reduction, "loss": loss,
        "loss_per_lead": loss if reduction == "mean" else loss / n,
        "loss_sum_estimated": loss * n if reduction == "mean" else loss,
        "output_sum": output_sum, "output_dtype": str(output_dtype), "peak_memory_mb": peak, "step_time_s": step_time,
        "forward_time_s": forward_time,
        "rest_time_s": (step_time - forward_time) if forward_time is not None else None,
        "flops_tflops": (local_flops_per_step / step_time / 1e12) if step_time and local_flops_per_step else 0.0,
        "load_data_time_s": load_time,
    }
    row.update(more)
    return row


def write_finetune_metrics(session, args, rows: Sequence[dict], lead_rows: Sequence[dict], facts: dict, flops,
                           lead: int, reduction: str, data_path: dict, extra: Optional[dict] = None):
    """``data_path``: the input-path switches of the run (pinning, non-blocking copies, double buffering and so on),
    recorded as they were resolved."""
    csv_path = os.path.abspath(args.metrics_csv) if args.metrics_csv else None
    if csv_path and rows:
        _write_csv(csv_path, FINETUNE_COLUMNS, rows)
    if args.memory_timeline_csv and lead_rows:
        _write_csv(args.memory_timeline_csv, LEAD_COLUMNS, lead_rows)
    json_path = json_path_for(args)
    if json_path is None:
        return
    pad = padding_facts(session.archi)
    meta = _run_metadata(session, args, len(rows))
    c = session.cfg
    record = {"script": "test_finetune.py"}
    for k in ("model_cfg", "task_type", "model_architecture", "model_type", "precision", "optimizer_config"):
        record[k] = meta[k]
    record["dp_size"] = session.dp
    for k in ("world_size", "ranks_per_dp", "wp_topo", "xfmr_wp_topo", "xfmr_sp_size", "tensor_parallel_size",
              "window_assignment_mode"):
        record[k] = meta[k]
    record.update({"lead_time": lead, "finetune_loss_reduction": reduction, "micro_batch_size": c.get("micro_batch_size"),
                   "use_fake_input": c.get("use_fake_input"), "fake_input_random": c.get("fake_input_random", True),
                   "fake_input_seed": c.get("fake_input_seed", 1234)})
    record.update(data_path)
    record["num_workers"] = int(c.get("num_workers", c.get("dataloader_num_workers", 1)))
    record["test_iter_num"] = len(rows)
    record["metrics_csv"] = csv_path
    record["parameter_count_by_rank"] = facts["parameter_count"]["post_wrap_local_parameter_counts_by_rank"]
    for k in ("peak_memory_last_by_rank", "step_time_last_by_rank", "boundary_offload_stats_by_rank"):
        record[k] = facts.get(k)
    for k in ("padding_policy", "padded_shape", "initial_padding", "patch_token_resolution",
              "transformer_token_resolution", "num_windows"):
        record[k] = pad[k]
    record.update(flops.as_metadata())
    record.update(extra or {})
    _write_json(json_path, record)
