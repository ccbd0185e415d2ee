"""Per-rank stdout / stderr redirection (reference: core/logging/logging.py:50-112).

Files: ``./log[/<embedding_parallel_type>]/<optimizer tag>_<seq|para>_dp_rank{d}_wp_rank{w}_wg{g}_sp{s}_tp{t}.txt``.
Only the first window-parallel rank of every data-parallel replica keeps its output; the others go to /dev/null. With
tensor parallelism the harnesses keep one rank per TP rank (``debug_log_wp_ranks``), since TP ranks hold different
parameter shards and their gradient reports differ (train_scripts/test_finetune.py:164-172 in the reference).
"""
from __future__ import annotations

import os
import sys


def optimizer_tag(optimizer_state_tuple) -> str:
    use_ddp, use_fsdp, zero_stage, use_dist_opt = optimizer_state_tuple
    if use_dist_opt:
        return "my_dist_optim"
    if use_fsdp:
        return "fsdp"
    if zero_stage is not None and zero_stage >= 0:
        return f"zero{zero_stage}"
    if use_ddp:
        return "ddp"
    return "rank"


def rank_log_path(manager, model_type, optimizer_state_tuple, embedding_parallel_type=None, root="./log") -> str:
    d = os.path.join(root, embedding_parallel_type) if embedding_parallel_type else root
    kind = "seq" if model_type == "sequential" else "para"
    name = (f"{optimizer_tag(optimizer_state_tuple)}_{kind}_dp_rank{manager.get_dp_rank()}_wp_rank{manager.get_wp_rank()}"
            f"_wg{manager.xfmr_window_group_rank}_sp{manager.xfmr_sp_rank}_tp{manager.xfmr_tp_rank}.txt")
    return os.path.join(d, name)


class _Tee:
    def __init__(self, stream):
        self.stream = stream

    def write(self, data):
        self.stream.write(data)
        self.stream.flush()

    def flush(self):
        self.stream.flush()


def debug_log_wp_ranks(manager, model_type, other_params) -> list:
    """Window-parallel ranks whose output is kept: rank 0, or with TP the first rank of every TP coordinate."""
    tp = int((other_params or {}).get("tensor_parallel_size", 1) or 1)
    if model_type not in ("parallel", "hybrid") or tp <= 1:
        return [0]
    if manager is not None and hasattr(manager, "xfmr_coord_to_wp_rank"):
        return [manager.xfmr_coord_to_wp_rank(0, 0, t) for t in range(tp)]
    return list(range(tp))


def set_dp_rank_print_redirect(manager, model_type, optimizer_state_tuple, embedding_parallel_type=None, quiet=False,
                               disable=False, root="./log", only_wp_ranks=(0,)):
    """Returns the path that now receives this rank's output (``None`` when nothing was redirected)."""
    if disable:
        return None
    if quiet or manager.get_wp_rank() not in set(only_wp_ranks):
        sink = open(os.devnull, "w")
        sys.stdout = sys.stderr = sink
        return os.devnull
    path = rank_log_path(manager, model_type, optimizer_state_tuple, embedding_parallel_type, root)
    os.makedirs(os.path.dirname(path), exist_ok=True)
    f = open(path, "a", buffering=1)
    sys.stdout = sys.stderr = _Tee(f)
    return path
