"""Which rank of the window dimension owns which Swin window.

Same results as the reference's ``get_window_indices`` (core/parallel/window_assignment.py:117-178) for its
six modes, computed in closed form with array arithmetic rather than by appending window by window:

``regular``                   owner = (jj % n) + (ii % m) * n
``ragged_round_robin``        owner = flat % (m*n); with n == 1 it degenerates to contiguous ragged rows
``terra_m1_regular``          contiguous blocks of nWh/m window rows
``terra_m1_ragged_row``       contiguous window rows, the first nWh % m ranks get one more
``terra_m1_ragged_row_major`` rank r owns flat windows [r*T//m, (r+1)*T//m)
``terra_m1_ragged_auto``      resolves to ``terra_m1_ragged_row_major``

The local window order of every activation tensor is row-major inside the rank's set.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import numpy as np

TERRA_M1_ASSIGNMENT_MODES = {
    "terra_m1_regular",
    "terra_m1_ragged_row",
    "terra_m1_ragged_row_major",
    "terra_m1_ragged_auto",
}
ALL_ASSIGNMENT_MODES = {"regular", "ragged_round_robin"} | TERRA_M1_ASSIGNMENT_MODES


def is_terra_m1_assignment_mode(mode: str) -> bool:
    return mode in TERRA_M1_ASSIGNMENT_MODES


def get_window_assignment_mode(manager) -> str:
    return getattr(manager, "window_assignment_mode", "regular")


def _row_counts(num_rows: int, m: int) -> np.ndarray:
    base, extra = divmod(num_rows, m)
    return np.array([base + (1 if r < extra else 0) for r in range(m)], dtype=np.int64)


def window_owner_map(num_windows_h: int, num_windows_w: int, wp_group_h: int, wp_group_w: int, mode: str = "regular") -> np.ndarray:
    """[nWh, nWw] int array: owning rank of every window."""
    if mode not in ALL_ASSIGNMENT_MODES:
        raise ValueError(f"Unsupported window_assignment_mode: {mode}")
    m, n = int(wp_group_h), int(wp_group_w)
    ii, jj = np.meshgrid(np.arange(num_windows_h), np.arange(num_windows_w), indexing="ij")
    flat = ii * num_windows_w + jj
    total = num_windows_h * num_windows_w
    if is_terra_m1_assignment_mode(mode):
        if n != 1:
            raise ValueError(f"{mode} requires xfmr_wp_topo=(m, 1), got ({m}, {n})")
        resolved = "terra_m1_ragged_row_major" if mode == "terra_m1_ragged_auto" else mode
        if resolved == "terra_m1_regular":
            if num_windows_h % m != 0:
                raise ValueError(f"terra_m1_regular requires num_windows_h={num_windows_h} divisible by m={m}")
            return ii // (num_windows_h // m)
        if resolved == "terra_m1_ragged_row":
            if num_windows_h < m:
                raise ValueError(f"terra_m1_ragged_row requires num_windows_h={num_windows_h} >= m={m}")
            ends = np.cumsum(_row_counts(num_windows_h, m))
            return np.searchsorted(ends, ii, side="right")
        if total < m:
            raise ValueError(f"terra_m1_ragged_row_major requires total_windows={total} >= m={m}")
        starts = (np.arange(m + 1) * total) // m
        return np.searchsorted(starts[1:], flat, side="right")
    if mode == "ragged_round_robin":
        if n == 1:
            ends = np.cumsum(_row_counts(num_windows_h, m))
            return np.searchsorted(ends, ii, side="right")
        return flat % (m * n)
    return (jj % n) + (ii % m) * n


def get_window_indices(num_windows_h, num_windows_w, wp_group_h, wp_group_w, mode="regular", debug_rank=None,
                       debug_global_rank=None):
    """Returns ``(rank_to_indices, global_to_local)`` exactly like the reference function of the same name."""
    owner = window_owner_map(num_windows_h, num_windows_w, wp_group_h, wp_group_w, mode)
    wp_size = int(wp_group_h) * int(wp_group_w)
    rank_to_indices: Dict[int, List[Tuple[int, int]]] = {r: [] for r in range(wp_size)}
    global_to_local: Dict[Tuple[int, int], Tuple[int, int]] = {}
    flat_owner = owner.reshape(-1)
    for flat_idx, r in enumerate(flat_owner.tolist()):
        ii, jj = divmod(flat_idx, num_windows_w)
        global_to_local[(ii, jj)] = (r, len(rank_to_indices[r]))
        rank_to_indices[r].append((ii, jj))
    return rank_to_indices, global_to_local


def flat_window_starts(num_windows_h: int, num_windows_w: int, m: int, mode: str) -> List[int]:
    """For the contiguous modes: ``starts`` with rank r owning flat windows [starts[r], starts[r+1]).

    Raises for modes whose ownership is not a contiguous flat range (``regular`` with m > 1 rows interleaved,
    round robin over n > 1)."""
    owner = window_owner_map(num_windows_h, num_windows_w, m, 1, mode).reshape(-1)
    if np.any(np.diff(owner) < 0):
        raise ValueError(f"window_assignment_mode={mode} does not give contiguous flat ranges for m={m}")
    counts = np.bincount(owner, minlength=m)
    return [0] + np.cumsum(counts).tolist()
