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


def _simulate_all_to_all(chunks_by_source, sizes_by_source, dest):
    """What rank ``dest`` receives: every source's chunk for it, in source order."""
    parts = []
    for src, (rows, sizes) in enumerate(zip(chunks_by_source, sizes_by_source)):
        start = sum(sizes[:dest])
        parts.append(rows[start:start + sizes[dest]])
    return torch.cat(parts, 0)


@pytest.mark.parametrize("seed,n_wg,sp,nWh,nWw,ws,batch", [
    (0, 3, 1, 3, 4, (4, 4), 1), (1, 4, 1, 2, 5, (4, 6), 2), (2, 2, 1, 4, 3, (5, 3), 1),      # odd window sides too
    (3, 2, 2, 3, 3, (4, 4), 1), (4, 3, 2, 2, 4, (2, 6), 2), (5, 2, 3, 3, 2, (3, 4), 1),
])
def test_shift_exchange_routes_for_arbitrary_owner_maps(seed, n_wg, sp, nWh, nWw, ws, batch):
    """The routed exchange of window-parallel attention, every rank simulated in one process with a RANDOM owner map:
    what a rank assembles must be exactly its owned shifted windows (q rows of its query slots, k / v rows of whole
    windows), each rank's send list must be what its peers expect, and the way back must put every output on its home
    row. Attention itself is replaced by the identity on the q rows."""
    from terra_b200.ops.attention import WindowGeometry, shifted_window_sources
    from terra_b200.parallel.context import _ShardedShiftExchangeAttnComm, _ShiftExchangeAttnComm

    rng = np.random.default_rng(seed)
    wh, ww = ws
    G, N = nWh * nWw, wh * ww
    sN = N // sp
    owner = np.concatenate([np.arange(n_wg), rng.integers(0, n_wg, G - n_wg)])        # every group owns something
    rng.shuffle(owner)
    windows_of = [np.nonzero(owner == g)[0] for g in range(n_wg)]
    world = n_wg * sp
    topo = Topology(wp_topo=(world, 1), xfmr_wp_topo=(n_wg, 1), xfmr_sp_size=sp, xfmr_tp_size=1)
    ctxs = []
    for r in range(world):
        c = ParallelContext(_Manager(topo, r), (wh, ww), (nWh * wh, nWw * ww), batch, "ragged_round_robin")
        c.owner, c.windows_of = owner, windows_of                                    # the random map replaces the mode's
        ctxs.append(c)
    torch.manual_seed(seed)
    X = torch.randn(batch, G, N, 3)                                                  # [q | k | v] as one column each
    src_win, src_tok, _ = shifted_window_sources(WindowGeometry(batch, nWh, nWw, wh, ww), True)

    def local_rows(r):
        g, s = divmod(r, sp)
        return X[:, windows_of[g], s * sN:(s + 1) * sN].reshape(-1, 3)

    def expected(r, slots):                                                          # shifted windows of the rank's group
        g, _ = divmod(r, sp)
        wins = windows_of[g]
        return X[:, src_win[wins][:, slots], src_tok[wins][:, slots]].reshape(-1, 3)

    dev = torch.device("cpu")
    if sp == 1:
        tabs = [_ShiftExchangeAttnComm(c, batch)._routes(dev) for c in ctxs]
        q_routes = kv_routes = tabs
        key = lambda t, k: t[k]
    else:
        tabs = [_ShardedShiftExchangeAttnComm(c, batch)._tables_for(True, dev) for c in ctxs]
        q_routes, kv_routes = [t["q"] for t in tabs], [t["kv"] for t in tabs]
        key = lambda t, k: t[k]
    rows = [local_rows(r) for r in range(world)]
    for routes, slots_of in ((q_routes, lambda r: slice((r % sp) * sN, (r % sp + 1) * sN)), (kv_routes, lambda r: slice(0, N))):
        sent = [rows[r].index_select(0, key(routes[r], "send_index")) for r in range(world)]
        sizes = [key(routes[r], "send_sizes") for r in range(world)]
        for d in range(world):
            got = _simulate_all_to_all(sent, sizes, d)
            assert got.shape[0] == sum(key(routes[d], "recv_sizes"))
            assert [sizes[s][d] for s in range(world)] == list(key(routes[d], "recv_sizes"))
            mine = torch.cat([rows[d], got], 0).index_select(0, key(routes[d], "assemble"))
            assert torch.equal(mine, expected(d, slots_of(d))), (d, "assembled windows differ from the definition")
    # the way back along the q routes: identity "attention" returns every q row to its home
    outs = [torch.cat([rows[r], _simulate_all_to_all(
        [rows[s].index_select(0, key(q_routes[s], "send_index")) for s in range(world)],
        [key(q_routes[s], "send_sizes") for s in range(world)], r)], 0).index_select(0, key(q_routes[r], "assemble"))
        for r in range(world)]
    returned = [outs[r].index_select(0, key(q_routes[r], "return_index")) for r in range(world)]
    back_sizes = [key(q_routes[r], "recv_sizes") for r in range(world)]
    for d in range(world):
        back = _simulate_all_to_all(returned, back_sizes, d)
        home = torch.cat([outs[d], back], 0).index_select(0, key(q_routes[d], "home"))
        assert torch.equal(home, rows[d]), (d, "an output did not return to its home row")
