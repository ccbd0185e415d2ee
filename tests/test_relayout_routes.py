"""The (rank, row) route tables of the general stripe <-> window relayout, checked on the CPU by simulating every rank:
pulling rows by the table must equal the definition (cut the global token grid into windows, keep this rank's windows,
token shard and tensor-parallel chunk), and the two directions must be inverse to each other. Covers ragged window
ownership, sequence parallelism and tensor parallelism (reference: core/parallel/layout_transform.py:107-173,244-263)."""
import numpy as np
import pytest
import torch

from terra_b200.parallel.context import ParallelContext
from terra_b200.parallel.rank_manager import Topology


class _Manager:
    """The attributes ParallelContext reads from a ParallelManager, without a process group."""

    def __init__(self, topo: Topology, wp_rank: int):
        self.topo = topo
        self.wp_size, self.wp_rank = topo.wp_size, wp_rank
        self.xfmr_wp_topo = topo.xfmr_wp_topo
        self.xfmr_window_group_size = topo.window_group_size
        self.xfmr_sp_size, self.xfmr_tp_size = topo.xfmr_sp_size, topo.xfmr_tp_size
        self.xfmr_window_group_rank, self.xfmr_sp_rank, self.xfmr_tp_rank = topo.wp_rank_to_xfmr_coord(wp_rank)
        self.window_parallel_group, self.window_parallel_ranks = None, list(range(topo.wp_size))

    def wp_rank_to_xfmr_coord(self, r):
        return self.topo.wp_rank_to_xfmr_coord(r)


@pytest.mark.parametrize("wp,xfmr,sp,tp,mode,Ht,Wt,ws,batch", [
    (4, (4, 1), 1, 1, "terra_m1_ragged_auto", 24, 40, 8, 1),       # 3 x 5 windows over 4 ranks: ragged, mid-row cuts
    (8, (8, 1), 1, 1, "terra_m1_ragged_auto", 96, 180, (8, 12), 1),   # 12 x 15 windows of 8 x 12 over 8 ranks
    (4, (1, 1), 2, 2, "regular", 32, 64, 8, 2),                    # token shards x tensor-parallel chunks, batch 2
    (8, (2, 1), 2, 2, "terra_m1_ragged_auto", 32, 64, 8, 1),       # 2 x 2 x 2
    (2, (1, 1), 1, 2, "regular", 24, 56, 8, 1),                    # 21 windows over 2 TP ranks: chunks of 11 and 10
])
def test_routes_reproduce_the_definition_and_invert_each_other(wp, xfmr, sp, tp, mode, Ht, Wt, ws, batch):
    topo = Topology(wp_topo=(wp, 1), xfmr_wp_topo=xfmr, xfmr_sp_size=sp, xfmr_tp_size=tp)
    ctxs = [ParallelContext(_Manager(topo, r), ws if isinstance(ws, tuple) else (ws, ws), (Ht, Wt), batch, mode) for r in range(wp)]
    C = 3
    torch.manual_seed(0)
    image = torch.randn(batch, Ht, Wt, C)
    h = Ht // wp
    stripes = [image[:, r * h:(r + 1) * h].reshape(-1, C) for r in range(wp)]
    win_bufs = []
    for r, p in enumerate(ctxs):
        (s2w_rank, s2w_row), _ = p.relayout_routes(batch)
        got = torch.stack([stripes[k][j] for k, j in zip(s2w_rank.tolist(), s2w_row.tolist())])
        # the definition: windows of the global grid, this rank's windows / token shard
        win = image.reshape(batch, p.nWh, p.wh, p.nWw, p.ww, C).permute(0, 1, 3, 2, 4, 5).reshape(batch, p.nWh * p.nWw, p.N, C)
        ids = torch.as_tensor(np.asarray(p._my_window_ids()), dtype=torch.long)
        want = win[:, ids][:, :, p.sp_rank * p.shardN:(p.sp_rank + 1) * p.shardN].reshape(-1, C)
        assert got.shape == want.shape and torch.equal(got, want), f"stripe -> windows differs on rank {r}"
        win_bufs.append(got)
    for r, p in enumerate(ctxs):
        _, (w2s_rank, w2s_row) = p.relayout_routes(batch)
        back = torch.stack([win_bufs[k][j] for k, j in zip(w2s_rank.tolist(), w2s_row.tolist())])
        assert torch.equal(back, stripes[r]), f"windows -> stripe differs on rank {r}"
