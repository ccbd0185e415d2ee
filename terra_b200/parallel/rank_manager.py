"""Rank algebra and process groups of the DP x (window group x SP x TP) layout.

``Topology`` is pure arithmetic (unit-testable without torch.distributed); ``ParallelManager`` adds the
process groups and keeps the attribute and method names that models, optimizer and entry points of the
reference read (core/rank_manager.py:6-396):

    global rank = dp * (mp * wp) + mp_rank * wp + wp_rank
    wp_rank     = wg * (sp * tp) + (sp_rank * tp + tp_rank   if tp_first
                                    tp_rank * sp + sp_rank   if sp_first)
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch.distributed as dist


@dataclass(frozen=True)
class Topology:
    dp_size: int = 1
    mp_size: int = 1
    wp_topo: Tuple[int, int] = (1, 1)
    xfmr_wp_topo: Optional[Tuple[int, int]] = None
    xfmr_sp_size: int = 1
    xfmr_tp_size: int = 1
    sp_tp_placement: str = "tp_first"

    def __post_init__(self):
        if self.xfmr_sp_size < 1:
            raise ValueError(f"xfmr_sp_size must be >= 1, got {self.xfmr_sp_size}")
        if self.xfmr_tp_size < 1:
            raise ValueError(f"tensor_parallel_size must be >= 1, got {self.xfmr_tp_size}")
        if self.sp_tp_placement not in ("tp_first", "sp_first"):
            raise ValueError(f"sp_tp_placement must be 'tp_first' or 'sp_first', got {self.sp_tp_placement}")
        if self.xfmr_wp_topo is None:
            object.__setattr__(self, "xfmr_wp_topo", tuple(self.wp_topo))
        if self.window_group_size * self.xfmr_sp_size * self.xfmr_tp_size != self.wp_size:
            raise ValueError(
                f"xfmr_wp_topo={self.xfmr_wp_topo} product times xfmr_sp_size={self.xfmr_sp_size} times "
                f"tensor_parallel_size={self.xfmr_tp_size} must equal wp_topo={self.wp_topo} product")

    @property
    def wp_size(self) -> int:
        return self.wp_topo[0] * self.wp_topo[1]

    @property
    def window_group_size(self) -> int:
        return self.xfmr_wp_topo[0] * self.xfmr_wp_topo[1]

    @property
    def world_size(self) -> int:
        return self.dp_size * self.mp_size * self.wp_size

    # ---- rank algebra
    def global_rank(self, dp_rank: int, mp_rank: int, wp_rank: int) -> int:
        return dp_rank * (self.mp_size * self.wp_size) + mp_rank * self.wp_size + wp_rank

    def split_rank(self, rank: int) -> Tuple[int, int, int]:
        denom = self.mp_size * self.wp_size
        rem = rank % denom
        return rank // denom, rem // self.wp_size, rem % self.wp_size

    def xfmr_coord_to_wp_rank(self, wg: int, sp: int, tp: int) -> int:
        if not 0 <= wg < self.window_group_size:
            raise ValueError(f"invalid window_group_rank={wg}")
        if not 0 <= sp < self.xfmr_sp_size:
            raise ValueError(f"invalid sp_rank={sp}")
        if not 0 <= tp < self.xfmr_tp_size:
            raise ValueError(f"invalid tp_rank={tp}")
        base = wg * (self.xfmr_sp_size * self.xfmr_tp_size)
        if self.sp_tp_placement == "tp_first":
            return base + sp * self.xfmr_tp_size + tp
        return base + tp * self.xfmr_sp_size + sp

    def wp_rank_to_xfmr_coord(self, wp_rank: int) -> Tuple[int, int, int]:
        if not 0 <= wp_rank < self.wp_size:
            raise ValueError(f"invalid wp_rank={wp_rank}")
        inner = self.xfmr_sp_size * self.xfmr_tp_size
        wg, r = divmod(wp_rank, inner)
        if self.sp_tp_placement == "tp_first":
            sp, tp = divmod(r, self.xfmr_tp_size)
        else:
            tp, sp = divmod(r, self.xfmr_sp_size)
        return wg, sp, tp

    def xfmr_coord_to_global_rank(self, dp: int, mp: int, wg: int, sp: int, tp: int) -> int:
        return self.global_rank(dp, mp, self.xfmr_coord_to_wp_rank(wg, sp, tp))

    # ---- group membership lists, in the deterministic creation order
    def dp_groups(self) -> List[List[int]]:
        return [[self.global_rank(d, m, w) for d in range(self.dp_size)]
                for m in range(self.mp_size) for w in range(self.wp_size)]

    def mp_groups(self) -> List[List[int]]:
        return [[self.global_rank(d, m, w) for m in range(self.mp_size)]
                for d in range(self.dp_size) for w in range(self.wp_size)]

    def wp_groups(self) -> List[List[int]]:
        return [[self.global_rank(d, m, w) for w in range(self.wp_size)]
                for d in range(self.dp_size) for m in range(self.mp_size)]

    def sp_groups(self) -> List[List[int]]:
        return [[self.xfmr_coord_to_global_rank(d, m, g, s, t) for s in range(self.xfmr_sp_size)]
                for d in range(self.dp_size) for m in range(self.mp_size)
                for g in range(self.window_group_size) for t in range(self.xfmr_tp_size)]

    def tp_groups(self) -> List[List[int]]:
        return [[self.xfmr_coord_to_global_rank(d, m, g, s, t) for t in range(self.xfmr_tp_size)]
                for d in range(self.dp_size) for m in range(self.mp_size)
                for g in range(self.window_group_size) for s in range(self.xfmr_sp_size)]

    def tp_param_groups(self) -> List[List[int]]:
        """Window group x SP at fixed TP rank (ranks that hold the same TP shard within one DP replica)."""
        return [[self.xfmr_coord_to_global_rank(d, m, g, s, t)
                 for g in range(self.window_group_size) for s in range(self.xfmr_sp_size)]
                for d in range(self.dp_size) for m in range(self.mp_size) for t in range(self.xfmr_tp_size)]

    def full_param_replica_groups(self) -> List[List[int]]:
        return [[self.global_rank(d, m, w) for d in range(self.dp_size) for w in range(self.wp_size)]
                for m in range(self.mp_size)]

    def tp_param_replica_groups(self) -> List[List[int]]:
        return [[self.xfmr_coord_to_global_rank(d, m, g, s, t) for d in range(self.dp_size)
                 for g in range(self.window_group_size) for s in range(self.xfmr_sp_size)]
                for m in range(self.mp_size) for t in range(self.xfmr_tp_size)]

    def window_group_groups(self) -> List[List[int]]:
        """Ranks that differ only in the window-group coordinate (peers of the shifted-window halo)."""
        return [[self.xfmr_coord_to_global_rank(d, m, g, s, t) for g in range(self.window_group_size)]
                for d in range(self.dp_size) for m in range(self.mp_size)
                for s in range(self.xfmr_sp_size) for t in range(self.xfmr_tp_size)]


def validate_node_aligned_wp_groups(wp_size: int, world_size: int) -> None:
    """WP groups may span nodes only in whole nodes (reference guard, core/rank_manager.py:99-126)."""
    if os.environ.get("TERRA_ALLOW_UNALIGNED_CROSS_NODE_WP", "0") == "1":
        return
    local_world = int(os.environ.get("LOCAL_WORLD_SIZE") or os.environ.get("NPROC_PER_NODE") or 0)
    if local_world <= 1 or wp_size <= 1:
        return
    if 0 < world_size <= local_world:
        return
    if local_world % wp_size == 0 or wp_size % local_world == 0:
        return
    raise RuntimeError(
        "[TERRA WARNING] unsupported cross-node window_parallel_group placement: "
        f"wp_size={wp_size}, local_world_size={local_world}, world_size={world_size}. "
        "Use a node-aligned wp_size, or set TERRA_ALLOW_UNALIGNED_CROSS_NODE_WP=1 for manual debugging.")


class ParallelManager:
    """Process groups of one run. All ranks must construct it with identical arguments."""

    def __init__(self, dp_size=1, mp_size=1, wp_topo=(1, 1), xfmr_wp_topo=None, domain_topo=(1, 1), rank=-1,
                 world_size=-1, device=None, window_assignment_mode="regular", xfmr_sp_size=1,
                 tensor_parallel_size=1, sp_tp_placement="tp_first"):
        self.topology = Topology(int(dp_size), int(mp_size), tuple(wp_topo),
                                 None if xfmr_wp_topo is None else tuple(xfmr_wp_topo), int(xfmr_sp_size),
                                 int(tensor_parallel_size), sp_tp_placement)
        t = self.topology
        self.rank = self.global_rank = rank
        self.world_size = world_size
        self.dp_size, self.mp_size, self.wp_size = t.dp_size, t.mp_size, t.wp_size
        validate_node_aligned_wp_groups(self.wp_size, world_size)
        self.xfmr_sp_size, self.xfmr_tp_size = t.xfmr_sp_size, t.xfmr_tp_size
        self.xfmr_window_group_size = t.window_group_size
        self.sp_tp_placement = sp_tp_placement
        self.data_wp_topo = tuple(wp_topo)
        self.data_wp_group_h, self.data_wp_group_w = self.data_wp_topo
        self.wp_group_h, self.wp_group_w = self.data_wp_topo
        self.xfmr_wp_topo = t.xfmr_wp_topo
        self.xfmr_wp_group_h, self.xfmr_wp_group_w = t.xfmr_wp_topo
        self.window_assignment_mode = window_assignment_mode
        self.num_windows_h = self.num_windows_w = -1
        self.domain_topo = domain_topo
        self.device = device

        self.dp_rank, self.mp_rank, self.wp_rank = t.split_rank(rank)
        self.xfmr_window_group_rank, self.xfmr_sp_rank, self.xfmr_tp_rank = t.wp_rank_to_xfmr_coord(self.wp_rank)

        # Every rank creates every group in the same total order.
        self.data_parallel_group, self.data_parallel_ranks = self._make(t.dp_groups())
        self.model_parallel_group, self.model_parallel_ranks = self._make(t.mp_groups())
        self.window_parallel_group, self.window_parallel_ranks = self._make(t.wp_groups())
        self.xfmr_sp_group, self.xfmr_sp_ranks = self._make(t.sp_groups())
        self.xfmr_tp_group, self.xfmr_tp_ranks = self._make(t.tp_groups())
        self.xfmr_tp_param_group, self.xfmr_tp_param_ranks = self._make(t.tp_param_groups())
        self.full_param_replica_group, self.full_param_replica_ranks = self._make(t.full_param_replica_groups())
        self.xfmr_tp_param_replica_group, self.xfmr_tp_param_replica_ranks = self._make(t.tp_param_replica_groups())
        self.xfmr_window_group, self.xfmr_window_group_ranks = self._make(t.window_group_groups())

        self.mp_group_size = len(self.model_parallel_ranks)
        self.dp_group_size = len(self.data_parallel_ranks)
        self.wp_group_size = len(self.window_parallel_ranks)
        self.domain_parallel_size = self.wp_group_size
        self._domain_group_idx = self.rank // self.domain_parallel_size
        self._domain_rank = self.rank % self.domain_parallel_size

    def _make(self, groups):
        mine, mine_ranks = None, None
        for ranks in groups:
            handle = dist.new_group(ranks=ranks)
            if self.rank in ranks:
                mine, mine_ranks = handle, list(ranks)
        if mine is None:
            raise RuntimeError(f"rank {self.rank} is in no group of {groups}")
        return mine, mine_ranks

    # ---- reference-compatible accessors
    def xfmr_coord_to_wp_rank(self, wg, sp, tp):
        return self.topology.xfmr_coord_to_wp_rank(wg, sp, tp)

    def wp_rank_to_xfmr_coord(self, wp_rank):
        return self.topology.wp_rank_to_xfmr_coord(wp_rank)

    def xfmr_coord_to_global_rank(self, dp, mp, wg, sp, tp):
        return self.topology.xfmr_coord_to_global_rank(dp, mp, wg, sp, tp)

    def update_window_info(self, num_windows_h, num_windows_w):
        self.num_windows_h, self.num_windows_w = num_windows_h, num_windows_w

    def get_rank(self):
        return self.rank

    def get_dp_rank(self):
        return self.dp_rank

    def get_mp_rank(self):
        return self.mp_rank

    def get_wp_rank(self):
        return self.wp_rank

    def get_dp_group_size(self):
        return self.dp_group_size

    def get_mp_group_size(self):
        return self.mp_group_size

    def get_wp_group_size(self):
        return self.wp_group_size

    def get_global_rank(self, dp_rank, mp_rank, wp_rank):
        return self.topology.global_rank(dp_rank, mp_rank, wp_rank)

    def domain_rank(self):
        return self._domain_rank

    def is_first_domain_rank(self):
        return self._domain_rank == 0

    def is_last_domain_rank(self):
        return self._domain_rank == self.domain_parallel_size - 1

    def get_neighbor_global_rank(self, group=None, dp_rank=None, mp_rank=None, wp_rank=None):
        """Previous / next rank of the (non-periodic) row-stripe decomposition, ``None`` at the ends."""
        base = self._domain_group_idx * self.domain_parallel_size
        prev_rank = base + self._domain_rank - 1 if self._domain_rank > 0 else None
        next_rank = base + self._domain_rank + 1 if self._domain_rank < self.domain_parallel_size - 1 else None
        return prev_rank, next_rank


class SingleProcessManager:
    """Stand-in with the ``ParallelManager`` surface for a run without ``torch.distributed`` (one GPU or CPU)."""

    def __init__(self, device=None, window_assignment_mode="regular"):
        self.topology = Topology()
        self.rank = self.global_rank = 0
        self.world_size = 1
        self.dp_size = self.mp_size = self.wp_size = 1
        self.xfmr_sp_size = self.xfmr_tp_size = self.xfmr_window_group_size = 1
        self.sp_tp_placement = "tp_first"
        self.data_wp_topo = self.xfmr_wp_topo = (1, 1)
        self.data_wp_group_h = self.data_wp_group_w = self.wp_group_h = self.wp_group_w = 1
        self.xfmr_wp_group_h = self.xfmr_wp_group_w = 1
        self.window_assignment_mode = window_assignment_mode
        self.num_windows_h = self.num_windows_w = -1
        self.device = device
        self.dp_rank = self.mp_rank = self.wp_rank = 0
        self.xfmr_window_group_rank = self.xfmr_sp_rank = self.xfmr_tp_rank = 0
        for name in ("data_parallel", "model_parallel", "window_parallel", "xfmr_sp", "xfmr_tp", "xfmr_tp_param",
                     "full_param_replica", "xfmr_tp_param_replica", "xfmr_window"):
            setattr(self, name + "_group", None)
            setattr(self, name + "_ranks", [0])
        self.mp_group_size = self.dp_group_size = self.wp_group_size = self.domain_parallel_size = 1

    def update_window_info(self, h, w):
        self.num_windows_h, self.num_windows_w = h, w

    def xfmr_coord_to_wp_rank(self, wg, sp, tp):
        return 0

    def wp_rank_to_xfmr_coord(self, wp_rank):
        return 0, 0, 0

    def get_rank(self):
        return 0

    get_dp_rank = get_mp_rank = get_wp_rank = get_rank

    def get_dp_group_size(self):
        return 1

    get_mp_group_size = get_wp_group_size = get_dp_group_size

    def get_global_rank(self, dp_rank, mp_rank, wp_rank):
        return 0

    def is_first_domain_rank(self):
        return True

    is_last_domain_rank = is_first_domain_rank

    def get_neighbor_global_rank(self, *a, **k):
        return None, None
