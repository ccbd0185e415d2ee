"""Window ownership: the reference's two unit tests plus a comparison of every mode against the reference's own
function when it is installed (tests/unit/test_window_assignment.py in the reference)."""
import numpy as np
import pytest

from terra_b200.parallel.window_assignment import (flat_window_starts, get_window_indices, window_owner_map)


def _flat_ids(rank_to_indices, num_windows_w):
    return [[ii * num_windows_w + jj for ii, jj in rank_to_indices[r]] for r in sorted(rank_to_indices)]


def test_terra_m1_ragged_auto_assigns_contiguous_balanced_chunks():
    rank_to_indices, global_to_local = get_window_indices(2, 5, 4, 1, mode="terra_m1_ragged_auto")
    assert _flat_ids(rank_to_indices, 5) == [[0, 1], [2, 3, 4], [5, 6], [7, 8, 9]]
    assert global_to_local[(0, 2)] == (1, 0)
    assert global_to_local[(1, 4)] == (3, 2)


def test_terra_m1_modes_reject_non_m1_topology():
    for mode in ("terra_m1_regular", "terra_m1_ragged_row", "terra_m1_ragged_row_major", "terra_m1_ragged_auto"):
        with pytest.raises(ValueError):
            get_window_indices(4, 4, 2, 2, mode=mode)


def test_regular_and_round_robin():
    owner = window_owner_map(4, 6, 2, 3, "regular")
    assert owner[0].tolist() == [0, 1, 2, 0, 1, 2] and owner[1].tolist() == [3, 4, 5, 3, 4, 5]
    rr = window_owner_map(2, 5, 2, 2, "ragged_round_robin").reshape(-1)
    assert rr.tolist() == [i % 4 for i in range(10)]
    rows = window_owner_map(5, 3, 2, 1, "ragged_round_robin")
    assert rows[:, 0].tolist() == [0, 0, 0, 1, 1]


def test_ragged_rows_and_starts():
    owner = window_owner_map(12, 15, 8, 1, "terra_m1_ragged_row")
    assert np.bincount(owner[:, 0]).tolist() == [2, 2, 2, 2, 1, 1, 1, 1]
    starts = flat_window_starts(12, 15, 8, "terra_m1_ragged_auto")
    assert starts[0] == 0 and starts[-1] == 180
    assert sorted(set(np.diff(starts).tolist())) == [22, 23]
    with pytest.raises(ValueError):
        flat_window_starts(4, 4, 2, "regular")


@pytest.mark.parametrize("mode,m,n", [("regular", 2, 2), ("regular", 4, 1), ("ragged_round_robin", 3, 1),
                                      ("ragged_round_robin", 2, 3), ("terra_m1_regular", 4, 1),
                                      ("terra_m1_ragged_row", 5, 1), ("terra_m1_ragged_row_major", 7, 1),
                                      ("terra_m1_ragged_auto", 8, 1)])
def test_matches_reference_when_installed(mode, m, n):
    from baseline import ref_import

    if not ref_import.available():
        pytest.skip("reference not installed")
    ref_import.enable()
    from core.parallel.window_assignment import get_window_indices as ref_fn

    nh, nw = (12, 18)
    a, b = get_window_indices(nh, nw, m, n, mode)
    ra, rb = ref_fn(nh, nw, m, n, mode)
    assert a == ra and b == rb
