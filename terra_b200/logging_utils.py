"""Per-rank stdout / stderr redirection (reference: core/logging/logging.py:50-112).

Files: ``./log[/<embedding_parallel_type>]/<optimizer tag>_<seq|para>_dp_rank{d}_wp_rank{w}_wg{g}_sp{s}_tp{t}.txt``.
Only the first window-parallel rank of every data-parallel replica keeps its output; the others go to /dev/null.
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


def set_dp_rank_print_redirect(manager, model_type, optimizer_state_tuple, embedding_parallel_type=None, quiet=False,
                               disable=False, root="./log"):
    """Returns the path that now receives this rank's output (``None`` when nothing was redirected)."""
    if disable:
        return None
    if quiet or manager.get_wp_rank() != 0:
        sink = open(os.devnull, "w")
        sys.stdout = sys.stderr = sink
        return os.devnull
    path = rank_log_path(manager, model_type, optimizer_state_tuple, embedding_parallel_type, root)
    os.makedirs(os.path.dirname(path), exist_ok=True)
    f = open(path, "a", buffering=1)
    sys.stdout = sys.stderr = _Tee(f)
    return path
