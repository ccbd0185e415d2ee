"""Per-rank view of the parallel layout: who owns which rows, windows, token shards and channel shards, and the
operators whose implementation depends on that (attention / MLP halves, stripe <-> window relayout, sampling-block
halos and distributed GroupNorm).

Layouts (reference semantics: core/parallel/layout_transform.py, core/rank_manager.py:216-246):

* conv stage: NHWC row stripes of the token grid, ``H / wp`` rows per window-parallel rank, non-periodic halos;
* transformer stage: window-major rows ``[B, windows of my window group (TP chunk), my token shard, C]``:
  window group ``g`` owns the windows that the assignment mode gives it, SP rank ``s`` the tokens
  ``[s*shardN, (s+1)*shardN)`` of each window, TP rank ``t`` the chunk ``[t*wpt, (t+1)*wpt)`` of the group's
  windows between blocks (activations) and the heads / hidden channels ``t`` inside blocks (parameters).

Attention across ranks: the peer-memory kernels when the owner map is contiguous (``fused_comm``); otherwise, and on
the collective back ends, a routed exchange of the pieces of the owned (shifted) windows (``_ShiftExchangeAttnComm``,
with token shards ``_ShardedShiftExchangeAttnComm``), the Ulysses all-to-all for token shards of one window group, or
the gather-everything oracle (``_PortableAttnComm``).

With one rank every method degenerates to local index permutations.
"""
from __future__ import annotations

import os

from typing import List, Optional

import numpy as np
import torch
import torch.nn.functional as TF

from ..ops import blocks as B
from ..ops.attention import WindowGeometry, shifted_window_sources, window_attention, window_attention_reference
from . import collectives as C
from .window_assignment import window_owner_map


class DomainComm:
    """Row-stripe helpers for the sampling blocks (halo rows, GroupNorm statistics)."""

    def __init__(self, group, ranks: Optional[List[int]], rank_in_group: int):
        self.group = group
        self.ranks = ranks or [0]
        self.world = len(self.ranks)
        self.idx = rank_in_group
        self.prev = self.ranks[self.idx - 1] if self.idx > 0 else None
        self.next = self.ranks[self.idx + 1] if self.idx < self.world - 1 else None

    # ---- CPU / portable
    def halo_exchange_cpu(self, x_nchw, halo: int):
        return C.halo_rows(x_nchw, halo, self.prev, self.next, self.group)

    def group_norm_cpu(self, x, groups, weight, bias, eps):
        """GroupNorm whose statistics span the stripes of all ranks (two-moment form, one all-reduce)."""
        Bn, Cn, H, W = x.shape
        xg = x.reshape(Bn, groups, -1)
        s = torch.stack([xg.sum(-1), (xg * xg).sum(-1)], dim=-1)
        s = C.all_reduce_sum(s, self.group)
        n = xg.shape[-1] * self.world
        mean = s[..., 0] / n
        var = (s[..., 1] / n - mean * mean).clamp_min(0)
        xn = (xg - mean[..., None]) * torch.rsqrt(var + eps)[..., None]
        return xn.reshape(Bn, Cn, H, W) * weight[None, :, None, None] + bias[None, :, None, None]

    # ---- CUDA: over peer memory when ``peer`` is attached (terra_b200.parallel.nvlink.PeerDomain), else collectives
    peer = None

    def all_reduce_small(self, t):
        if self.peer is not None and t.is_cuda:
            return self.peer.all_reduce_small(t)
        return C.all_reduce_(t.clone(), self.group)

    def exchange_rows(self, x):
        """Boundary rows of the neighbours' stripes: ``(row above, row below)`` as ``[B, 1, W, C]`` tensors, ``None``
        at the global edges (the convolution then sees zeros there: non-periodic)."""
        top = x[:, :1]
        bot = x[:, -1:]
        if self.peer is not None and x.is_cuda:
            return self.peer.exchange_rows(top, bot)
        recv_prev, recv_next = C._exchange(top.contiguous(), bot.contiguous(), self.prev, self.next, self.group)
        return recv_prev, recv_next

    def fold_halo_grad(self, dxp, H, W):
        """dxp: [B, H+2, W+2, C] gradient of the zero/halo padded input -> gradient of the local rows, with the
        halo rows' gradients sent back to their owners."""
        if self.peer is not None and dxp.is_cuda:
            # my padded row 0 is the previous rank's last row, my padded row H + 1 the next rank's first row
            from_prev, from_next = self.peer.exchange_rows(dxp[:, 0:1, 1:W + 1], dxp[:, H + 1:H + 2, 1:W + 1])
            gx = dxp[:, 1:H + 1, 1:W + 1].contiguous()
            if from_prev is not None:
                gx[:, 0:1] += from_prev
            if from_next is not None:
                gx[:, H - 1:H] += from_next
            return gx
        g = dxp[:, :, 1:W + 1].permute(0, 3, 1, 2).contiguous()
        gx = C._HaloRows.backward(_Ctx((1, self.prev, self.next, self.group)), g)[0]
        return gx.permute(0, 2, 3, 1)


class _Ctx:
    """Minimal stand-in for an autograd context when a Function's forward/backward is used as a plain routine."""

    def __init__(self, p=None):
        self.p = p


class ParallelContext:
    def __init__(self, manager=None, window_size=(8, 8), token_hw=(0, 0), batch=1, window_assignment_mode="regular"):
        self.manager = manager
        self.wh, self.ww = int(window_size[0]), int(window_size[1])
        self.Ht, self.Wt = int(token_hw[0]), int(token_hw[1])
        if self.Ht % self.wh or self.Wt % self.ww:
            raise ValueError(f"token grid {(self.Ht, self.Wt)} must be divisible by window {(self.wh, self.ww)}")
        self.nWh, self.nWw = self.Ht // self.wh, self.Wt // self.ww
        self.B = batch
        m = manager
        self.world = m.wp_size if m is not None else 1
        self.wp_rank = m.wp_rank if m is not None else 0
        self.n_wg = m.xfmr_window_group_size if m is not None else 1
        self.sp = m.xfmr_sp_size if m is not None else 1
        self.tp = m.xfmr_tp_size if m is not None else 1
        self.wg_rank = m.xfmr_window_group_rank if m is not None else 0
        self.sp_rank = m.xfmr_sp_rank if m is not None else 0
        self.tp_rank = m.xfmr_tp_rank if m is not None else 0
        self.mode = window_assignment_mode
        topo = m.xfmr_wp_topo if m is not None else (1, 1)
        owner = window_owner_map(self.nWh, self.nWw, topo[0], topo[1], self.mode).reshape(-1)
        self.owner = owner
        self.windows_of = [np.nonzero(owner == g)[0] for g in range(self.n_wg)]      # flat ids, row-major
        counts = [len(w) for w in self.windows_of]
        self.contiguous = all(len(w) == 0 or (w[-1] - w[0] + 1 == len(w)) for w in self.windows_of) and \
            all(self.windows_of[g][0] == sum(counts[:g]) for g in range(self.n_wg) if counts[g])
        self.win_start = [0] + np.cumsum(counts).tolist()
        self.N = self.wh * self.ww
        self.shardN = (self.N + self.sp - 1) // self.sp
        if self.N % self.sp != 0:
            raise ValueError(f"window tokens {self.N} must be divisible by xfmr_sp_size {self.sp}")
        self.nW_group = counts[self.wg_rank]
        self.wpt = (self.nW_group + self.tp - 1) // self.tp                            # windows per TP rank
        self.tp_sizes_windows = [max(0, min(self.wpt, self.nW_group - t * self.wpt)) for t in range(self.tp)]
        self.dom = DomainComm(m.window_parallel_group if m is not None else None,
                              m.window_parallel_ranks if m is not None else None, self.wp_rank)
        self.fused_comm = None     # peer-memory (NVLink) implementation, attached by terra_b200.parallel.nvlink
        # stripe <-> window relayout is a local permutation when every rank's windows are exactly the windows of
        # its own row stripe (no token sharding, no TP chunking)
        self.local_relayout = self.world == 1
        if self.world > 1 and self.sp == 1 and self.tp == 1 and self.nWh % self.world == 0:
            per = (self.nWh // self.world) * self.nWw
            self.local_relayout = all(
                len(self.windows_of[g]) == per and self.windows_of[g][0] == g * per and self.windows_of[g][-1] == (g + 1) * per - 1
                for g in range(self.n_wg))

    # ------------------------------------------------------------------ geometry
    def geometry(self, batch: int, tp_chunked: bool = False) -> WindowGeometry:
        """``tp_chunked``: the q/k/v rows come out of the fused all-gather GEMM, i.e. as the concatenation of the
        tensor-parallel ranks' ``[B, windows per rank, tokens]`` chunks instead of ``[B, windows of the group, tokens]``."""
        return WindowGeometry(batch, self.nWh, self.nWw, self.wh, self.ww, list(self.win_start), self.wg_rank, self.sp,
                              self.sp_rank, self.tp if tp_chunked else 1)

    def rows_between_blocks(self, batch: int) -> int:
        return batch * self.tp_sizes_windows[self.tp_rank] * self.shardN

    # ------------------------------------------------------------------ transformer halves
    def attention_half(self, x, mod):
        batch = self._batch_of(x)
        geo = self.geometry(batch)
        comm = self._attn_comm(batch)
        if self.sp == 1 and self.tp == 1 and (comm is None or getattr(comm, "fused", False)):
            return B.attention_half(x, mod, geo, mod.shifted, comm)
        tpc = getattr(self, "tp_comm", None)
        if (self.tp > 1 and tpc is not None and x.is_cuda and (comm is None or getattr(comm, "fused", False))
                and self.N <= B.MAX_KERNEL_WINDOW_TOKENS):
            # both collectives of the tensor-parallel attention half run inside the GEMMs over NVLink peer memory
            from ..ops.tp_fused import tp_attention_half

            return tp_attention_half(x, mod, self.geometry(batch, tp_chunked=True), comm, tpc,
                                     batch * self.wpt * self.shardN, ragged=self.nW_group % self.tp != 0)
        return self._attention_half_factorized(x, mod, geo, batch)

    def mlp_half(self, x, mod):
        if self.tp == 1:
            return B.mlp_half(x, mod)
        return self._mlp_half_tp(x, mod)

    def _batch_of(self, x) -> int:
        per = self.tp_sizes_windows[self.tp_rank] * self.shardN
        return x.shape[0] // max(per, 1)

    def _attn_comm(self, batch):
        if self.n_wg * self.sp == 1:
            return None
        if self.fused_comm is not None and self.contiguous:
            return self.fused_comm
        if self.n_wg == 1 and self.sp > 1 and os.environ.get("TERRA_SP_BASELINE", "ulysses") == "ulysses":
            return _UlyssesAttnComm(self, batch)
        if self.n_wg > 1 and os.environ.get("TERRA_WP_BASELINE", "exchange") == "exchange":
            return self._cached_comm(_ShiftExchangeAttnComm if self.sp == 1 else _ShardedShiftExchangeAttnComm, batch)
        return _PortableAttnComm(self, batch)

    def _cached_comm(self, cls, batch):
        """One communicator per batch size: its route tables are built once."""
        cache = self.__dict__.setdefault("_comm_cache", {})
        if (cls, batch) not in cache:
            cache[(cls, batch)] = cls(self, batch)
        return cache[(cls, batch)]

    # ---- factorised SP / TP halves on portable collectives (CPU oracle path and the NCCL baseline)
    def _tp_sizes_rows(self, batch):
        return [batch * n * self.shardN for n in self.tp_sizes_windows]

    def _ag_tp(self, x, batch):
        if self.tp == 1:
            return x
        # rows are [B, windows, tokens]: gather along windows, batch stays outermost
        per = [n * self.shardN for n in self.tp_sizes_windows]
        xs = x.reshape(batch, per[self.tp_rank], -1).transpose(0, 1)
        full = C.all_gather_rows(xs, self.manager.xfmr_tp_group, per)
        return full.transpose(0, 1).reshape(batch * sum(per), -1)

    def _rs_tp(self, x, batch):
        if self.tp == 1:
            return x
        per = [n * self.shardN for n in self.tp_sizes_windows]
        xs = x.reshape(batch, sum(per), -1).transpose(0, 1)
        mine = C.reduce_scatter_rows(xs, self.manager.xfmr_tp_group, per)
        return mine.transpose(0, 1).reshape(batch * per[self.tp_rank], -1)

    def _lin(self, x, lin, residual=None):
        if x.is_cuda:
            return B.linear(x.contiguous(), lin, residual)
        y = TF.linear(x, lin.weight, lin.bias)
        return y if residual is None else y + residual

    def _ln(self, x, norm):
        if x.is_cuda:
            return _LayerNormFn.apply(x.contiguous(), norm.weight, norm.bias)
        return TF.layer_norm(x, (x.shape[-1],), norm.weight, norm.bias, B.LN_EPS)

    def _attention_half_factorized(self, x, mod, geo, batch):
        a = mod.attn
        xn = self._ln(x, mod.norm1)
        xa = self._ag_tp(xn, batch)
        qkv = torch.cat([self._lin(xa, a.q_linear), self._lin(xa, a.k_linear), self._lin(xa, a.v_linear)], dim=-1)
        comm = self._attn_comm(batch)
        o = window_attention(qkv.contiguous(), geo, a.num_heads, mod.shifted, a.bias_table(), mod.use_attn_mask, a.scale,
                             comm)
        part = self._lin(o, a.proj)
        y = self._rs_tp(part, batch)
        if hasattr(a, "proj_bias"):
            y = y + a.proj_bias.to(y.dtype)
        return x + y

    def _mlp_half_tp(self, x, mod):
        batch = self._batch_of(x)
        tpc = getattr(self, "tp_comm", None)
        if tpc is not None and x.is_cuda:
            # fc1 / fc2 with their all-gather / reduce-scatter fused into the GEMMs over NVLink peer memory
            from ..ops.tp_fused import tp_mlp_half

            return tp_mlp_half(x, mod, tpc, batch * self.wpt * self.shardN)
        xn = self._ln(x, mod.norm2)
        xa = self._ag_tp(xn, batch)
        h = self._lin(xa, mod.linear1)
        h = TF.gelu(h.float()).to(h.dtype) if h.is_cuda else TF.gelu(h)
        part = self._lin(h, mod.linear2)
        y = self._rs_tp(part, batch)
        return x + y + mod.bias2.to(y.dtype)

    # ------------------------------------------------------------------ stripe <-> window relayout
    def _peer_relayout(self, x):
        """The peer-memory implementation, when this rank's group has one and the tensor lives on a GPU."""
        peer = getattr(self.dom, "peer", None)
        return peer if (peer is not None and x.is_cuda and self.world > 1) else None

    def relayout_routes(self, batch):
        """Index tables of the general relayout, both directions: for every row of this rank's destination buffer,
        the window-parallel rank that holds the token and the row inside that rank's source buffer (the closed-form
        counterpart of the reference's route tables, core/parallel/layout_transform.py:67-87,338-376). Returns
        ``((rank, row) for stripe -> windows, (rank, row) for windows -> stripe)`` as int32 numpy arrays."""
        key = ("routes", batch)
        cache = self.__dict__.setdefault("_cache", {})
        if key in cache:
            return cache[key]
        sizes, img_pos = self._relayout_table(batch)          # image-major token -> position in the ranks' concatenation
        img_pos = img_pos.numpy()
        bounds = np.cumsum([0] + list(sizes))
        h = self.Ht // self.world
        # windows -> stripe: my stripe rows are image-major tokens (b, gh in my stripe, gw)
        tok = np.arange(batch * self.Ht * self.Wt, dtype=np.int64).reshape(batch, self.Ht, self.Wt)
        mine = tok[:, self.wp_rank * h:(self.wp_rank + 1) * h].reshape(-1)
        pos = img_pos[mine]
        w2s_rank = (np.searchsorted(bounds, pos, side="right") - 1).astype(np.int32)
        w2s_row = (pos - bounds[w2s_rank]).astype(np.int32)
        # stripe -> windows: invert for my window-major rows; a token's stripe rank is its image row // h
        lo, hi = bounds[self.wp_rank], bounds[self.wp_rank + 1]
        inv = np.full(hi - lo, -1, dtype=np.int64)
        sel = np.nonzero((img_pos >= lo) & (img_pos < hi))[0]
        inv[img_pos[sel] - lo] = sel                          # my row -> image-major token id
        b = inv // (self.Ht * self.Wt)
        rem = inv % (self.Ht * self.Wt)
        gh, gw = rem // self.Wt, rem % self.Wt
        s2w_rank = (gh // h).astype(np.int32)
        s2w_row = ((b * h + gh % h) * self.Wt + gw).astype(np.int32)
        pad = inv < 0                                          # rows of zero-padded windows (ragged TP chunks) have no source
        s2w_rank[pad] = self.wp_rank
        s2w_row[pad] = 0
        cache[key] = ((s2w_rank, s2w_row), (w2s_rank, w2s_row))
        return cache[key]

    def _routes_on(self, batch, device):
        key = ("routes_dev", batch, str(device))
        cache = self.__dict__.setdefault("_cache", {})
        if key not in cache:
            (a, b), (c, d) = self.relayout_routes(batch)
            cache[key] = tuple(torch.from_numpy(t).to(device) for t in (a, b, c, d))
        return cache[key]

    def stripe_to_windows(self, x):
        """NHWC row stripe ``[B, Ht/wp, Wt, C]`` -> this rank's window-major rows."""
        Bn, h, W, Cn = x.shape
        if self.local_relayout and self.world > 1:
            win = x.reshape(Bn, h // self.wh, self.wh, self.nWw, self.ww, Cn).permute(0, 1, 3, 2, 4, 5)
            return win.reshape(-1, Cn).contiguous()
        peer = self._peer_relayout(x)
        if peer is not None:
            s2w_rank, s2w_row, w2s_rank, w2s_row = self._routes_on(Bn, x.device)
            return _PeerRelayoutFn.apply(x.reshape(-1, Cn), peer, s2w_rank, s2w_row, w2s_rank, w2s_row)
        if self.world == 1:
            full = x
        else:
            rows = C.all_gather_rows(x.permute(1, 0, 2, 3).contiguous(), self.manager.window_parallel_group, None)
            full = rows.permute(1, 0, 2, 3)
        win = full.reshape(Bn, self.nWh, self.wh, self.nWw, self.ww, Cn).permute(0, 1, 3, 2, 4, 5)
        win = win.reshape(Bn, self.nWh * self.nWw, self.N, Cn)
        if self.world == 1:
            return win.reshape(-1, Cn).contiguous()
        ids = torch.as_tensor(self._my_window_ids(), device=x.device)
        mine = win[:, ids][:, :, self.sp_rank * self.shardN:(self.sp_rank + 1) * self.shardN]
        return mine.reshape(-1, Cn).contiguous()

    def _my_window_ids(self):
        w = self.windows_of[self.wg_rank]
        t0 = self.tp_rank * self.wpt
        return w[t0:t0 + self.tp_sizes_windows[self.tp_rank]]

    def windows_to_stripe(self, rows, batch):
        """Inverse of ``stripe_to_windows``."""
        Cn = rows.shape[-1]
        if self.local_relayout:
            nh = self.nWh // self.world
            win = rows.reshape(batch, nh, self.nWw, self.wh, self.ww, Cn).permute(0, 1, 3, 2, 4, 5)
            return win.reshape(batch, nh * self.wh, self.Wt, Cn).contiguous()
        m = self.manager
        peer = self._peer_relayout(rows)
        if peer is not None:
            s2w_rank, s2w_row, w2s_rank, w2s_row = self._routes_on(batch, rows.device)
            out = _PeerRelayoutFn.apply(rows, peer, w2s_rank, w2s_row, s2w_rank, s2w_row)
            return out.reshape(batch, self.Ht // self.world, self.Wt, Cn)
        sizes, index = self._relayout_table(batch)
        allrows = C.all_gather_rows(rows.contiguous(), m.window_parallel_group, sizes)
        full = allrows[index.to(rows.device)]                                            # [B*Ht*Wt, C] image-major
        full = full.reshape(batch, self.Ht, self.Wt, Cn)
        h = self.Ht // self.world
        return full[:, self.wp_rank * h:(self.wp_rank + 1) * h].contiguous()

    def _relayout_table(self, batch):
        """Row counts of every WP rank's window-major buffer and, for every image-major token, its position in
        the concatenation of those buffers."""
        key = ("relayout", batch)
        cache = self.__dict__.setdefault("_cache", {})
        if key in cache:
            return cache[key]
        m = self.manager
        nW, N = self.nWh * self.nWw, self.N
        pos = np.full((batch, nW, N), -1, dtype=np.int64)
        sizes, cursor = [], 0
        for wp in range(self.world):
            g, s, t = m.wp_rank_to_xfmr_coord(wp)
            wins = self.windows_of[g]
            wpt = (len(wins) + self.tp - 1) // self.tp
            mine = wins[t * wpt:min(len(wins), (t + 1) * wpt)]
            n = batch * len(mine) * self.shardN
            local = cursor + np.arange(n).reshape(batch, len(mine), self.shardN)
            pos[:, mine, s * self.shardN:(s + 1) * self.shardN] = local
            sizes.append(n)
            cursor += n
        img = pos.reshape(batch, self.nWh, self.nWw, self.wh, self.ww).transpose(0, 1, 3, 2, 4).reshape(-1)
        cache[key] = (sizes, torch.from_numpy(img))
        return cache[key]


_LayerNormFn = B.LayerNormFn


class _PeerRelayoutFn(torch.autograd.Function):
    """Relayout as a gather over peer memory: every destination row has exactly one source row on one rank, so the
    forward pulls the rows by a (rank, row) table and the backward pulls the gradient rows by the opposite table. The
    source is staged in symmetric memory; one barrier makes every rank's staging complete before the pulls."""

    @staticmethod
    def forward(ctx, x, peer, f_rank, f_row, b_rank, b_row):
        ctx.peer, ctx.tables = peer, (b_rank, b_row)
        ctx.src_rows = x.shape[0]
        return peer.gather_rows(x, f_rank, f_row)

    @staticmethod
    def backward(ctx, g):
        b_rank, b_row = ctx.tables
        out = ctx.peer.gather_rows(g.contiguous(), b_rank, b_row)
        assert out.shape[0] == ctx.src_rows
        return out, None, None, None, None, None


class _PortableAttnComm:
    """Window attention across window groups / token shards using only portable collectives: every rank of the
    (window group x SP) set gathers all q/k/v rows, evaluates the windows and keeps the outputs whose home
    rows it owns. Quadratically wasteful - it exists as the semantic oracle for gloo ranks and as the NCCL
    baseline; the peer-memory kernel path replaces it on NVLink."""

    fused = False

    def __init__(self, pctx: ParallelContext, batch: int):
        self.p = pctx
        self.batch = batch
        self.world = pctx.n_wg * pctx.sp

    def window_attention_portable(self, qkv, geo, num_heads, shifted, bias_table, use_mask, scale):
        p, m = self.p, self.p.manager
        Bn, N, sN = self.batch, p.N, p.shardN
        C3 = qkv.shape[-1]
        group, ranks = m.xfmr_tp_param_group, m.xfmr_tp_param_ranks            # (wg, sp) at my TP rank, wg-major
        sizes = []
        for g in range(p.n_wg):
            for s in range(p.sp):
                sizes.append(Bn * len(p.windows_of[g]) * sN)
        allrows = C.all_gather_rows(qkv.contiguous(), group, sizes)
        nW = p.nWh * p.nWw
        pos = np.full((Bn, nW, N), -1, dtype=np.int64)
        cursor = 0
        for g in range(p.n_wg):
            wins = p.windows_of[g]
            for s in range(p.sp):
                n = Bn * len(wins) * sN
                pos[:, wins, s * sN:(s + 1) * sN] = cursor + np.arange(n).reshape(Bn, len(wins), sN)
                cursor += n
        index = torch.from_numpy(pos.reshape(-1)).to(qkv.device)
        full = allrows[index].reshape(Bn, nW, N, C3)
        gfull = WindowGeometry(Bn, p.nWh, p.nWw, p.wh, p.ww)
        out = window_attention_reference(full, gfull, num_heads, shifted, bias_table, use_mask, scale)
        ids = torch.as_tensor(p.windows_of[p.wg_rank], device=qkv.device)
        mine = out[:, ids][:, :, p.sp_rank * sN:(p.sp_rank + 1) * sN]
        return mine.reshape(-1, C3 // 3)


class _ShiftExchangeAttnComm(_PortableAttnComm):
    """Window attention across window groups for ANY ownership map (contiguous or not), without gathering everything:
    the shifted window ``g`` is computed by the owner of window ``g``, which pulls the pieces of it that live in other
    windows - the role of the reference's quadrant exchange (core/window_parallel.py:26-266, point-to-point sends of the
    window corners along routes derived from the owner map). Here the routes are index tables over token rows: one
    all-to-all-v brings the foreign rows of every owned shifted window, the windows are then local (unshifted attention
    for the interior ones, which takes the fast kernel on a GPU; the windows on the frame's last row / column, whose
    tokens wrap around, with the region mask), and one all-to-all-v along the reversed routes returns the outputs to
    their home rows. Unshifted blocks need no communication. Token shards (SP > 1) stay on the gather / all-to-all
    baselines."""

    def __init__(self, pctx: "ParallelContext", batch: int):
        super().__init__(pctx, batch)
        self._tables = {}

    def _routes(self, device):
        key = str(device)
        if key in self._tables:
            return self._tables[key]
        p, Bn, N = self.p, self.batch, self.p.N
        gfull = WindowGeometry(Bn, p.nWh, p.nWw, p.wh, p.ww)
        src_win, src_tok, reg = (t.numpy() for t in shifted_window_sources(gfull, True))       # [nW, N]
        owner = np.asarray(p.owner)
        local_idx = np.zeros(owner.shape[0], dtype=np.int64)
        counts = []
        for g in range(p.n_wg):
            local_idx[p.windows_of[g]] = np.arange(len(p.windows_of[g]))
            counts.append(len(p.windows_of[g]))
        me = p.wg_rank

        def rows_of(rank_windows_count, b, wl, t):          # row of (batch b, local window wl, token t) on a rank
            return (b * rank_windows_count + wl) * N + t

        b_idx = np.arange(Bn)[:, None, None]
        # what I need: for my shifted windows, the source rank / row of every token, in (b, window, token) order
        mine = np.asarray(p.windows_of[me])
        s_rank = owner[src_win[mine]]                                                     # [nWl, N]
        s_row = rows_of(np.asarray(counts)[s_rank][None], b_idx, local_idx[src_win[mine]][None], src_tok[mine][None])
        s_rank_b = np.broadcast_to(s_rank[None], s_row.shape).reshape(-1)                 # [Bn * nWl * N]
        s_row = s_row.reshape(-1)
        n_mine = s_row.shape[0]
        recv_sizes = [int(((s_rank_b == r) & (r != me)).sum()) for r in range(p.n_wg)]
        recv_start = np.concatenate([[0], np.cumsum(recv_sizes)])
        assemble = np.empty(n_mine, dtype=np.int64)
        local = s_rank_b == me
        assemble[local] = s_row[local]
        for r in range(p.n_wg):
            if r == me:
                continue
            sel = s_rank_b == r
            assemble[sel] = n_mine_rows(self, me) + recv_start[r] + np.arange(int(sel.sum()))
        # what the others need from me, each in the destination's (b, window, token) order
        send_index, send_sizes = [], []
        for d in range(p.n_wg):
            if d == me or counts[d] == 0:
                send_sizes.append(0)
                continue
            theirs = np.asarray(p.windows_of[d])
            from_me = owner[src_win[theirs]] == me                                        # [nWd, N]
            rows = rows_of(counts[me], b_idx, local_idx[src_win[theirs]][None], src_tok[theirs][None])
            pick = np.broadcast_to(from_me[None], rows.shape).reshape(-1)
            send_index.append(rows.reshape(-1)[pick])
            send_sizes.append(int(pick.sum()))
        send_index = np.concatenate(send_index) if send_index else np.zeros(0, dtype=np.int64)
        # the way back: the rows I received return to their sources in the order they came; my home rows are then
        # either rows I computed myself or rows of the returned chunk, which arrives in my send order
        return_index = np.concatenate([np.nonzero(s_rank_b == r)[0] for r in range(p.n_wg) if r != me] or
                                      [np.zeros(0, dtype=np.int64)])
        home = np.full(n_mine_rows(self, me), -1, dtype=np.int64)
        home[s_row[local]] = np.nonzero(local)[0]
        home[send_index] = n_mine + np.arange(send_index.shape[0])
        if (home < 0).any():
            raise RuntimeError("shift exchange: a home row has no producer (owner map and routes disagree)")
        edge = np.array([i for i, g in enumerate(mine) if (reg[g] != reg[g][0]).any()], dtype=np.int64)
        inner = np.array([i for i, g in enumerate(mine) if not (reg[g] != reg[g][0]).any()], dtype=np.int64)
        to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
        t = dict(send_index=to(send_index), send_sizes=send_sizes, recv_sizes=recv_sizes, assemble=to(assemble),
                 return_index=to(return_index), home=to(home), edge=to(edge), inner=to(inner),
                 edge_reg=to(reg[mine[edge]]) if edge.size else None, windows=len(mine))
        self._tables[key] = t
        return t

    def window_attention_portable(self, qkv, geo, num_heads, shifted, bias_table, use_mask, scale):
        from ..ops.attention import attention_core_reference, relative_position_index

        p, Bn, N = self.p, self.batch, self.p.N
        C3 = qkv.shape[-1]
        nWl = len(p.windows_of[p.wg_rank])
        plain = WindowGeometry(Bn, nWl, 1, p.wh, p.ww)
        if not shifted:
            return window_attention(qkv.contiguous(), plain, num_heads, False, bias_table, use_mask, scale, None)
        t = self._routes(qkv.device)
        group = p.manager.xfmr_tp_param_group
        got = C.all_to_all_rows(qkv.index_select(0, t["send_index"]), group, t["send_sizes"], t["recv_sizes"])
        sq = torch.cat([qkv, got], 0).index_select(0, t["assemble"])                     # my shifted windows, complete
        if not use_mask or t["edge"].numel() == 0:
            o = window_attention(sq, plain, num_heads, False, bias_table, use_mask, scale, None)
        else:
            sq4 = sq.reshape(Bn, nWl, N, C3)
            o4 = sq.new_zeros(Bn, nWl, N, C3 // 3)
            if t["inner"].numel():
                xi = sq4.index_select(1, t["inner"]).reshape(-1, C3)
                oi = window_attention(xi, WindowGeometry(Bn, int(t["inner"].numel()), 1, p.wh, p.ww), num_heads, False,
                                      bias_table, use_mask, scale, None)
                o4 = o4.index_copy(1, t["inner"], oi.reshape(Bn, -1, N, C3 // 3).to(o4.dtype))
            ne = int(t["edge"].numel())
            hd = C3 // 3 // num_heads
            xe = sq4.index_select(1, t["edge"]).reshape(Bn * ne, N, 3, num_heads, hd)
            q, k, v = (xe[:, :, i].permute(0, 2, 1, 3) for i in range(3))                 # [Bn*ne, heads, N, hd]
            bias = None
            if bias_table is not None:
                idx = relative_position_index(p.wh, p.ww).to(bias_table.device)
                bias = bias_table[idx.reshape(-1)].reshape(N, N, num_heads).permute(2, 0, 1).to(q.dtype)
            reg = t["edge_reg"]
            mask = ((reg[:, :, None] != reg[:, None, :]).to(q.dtype) * -100.0).repeat(Bn, 1, 1)
            oe = attention_core_reference(q, k, v, scale, bias, mask).permute(0, 2, 1, 3).reshape(Bn, ne, N, C3 // 3)
            o4 = o4.index_copy(1, t["edge"], oe.to(o4.dtype))
            o = o4.reshape(-1, C3 // 3)
        back = C.all_to_all_rows(o.index_select(0, t["return_index"]), group, t["recv_sizes"], t["send_sizes"])
        return torch.cat([o, back], 0).index_select(0, t["home"])


def n_mine_rows(comm, rank) -> int:
    """Rows of q/k/v a rank holds: batch x its windows x the window's tokens."""
    return comm.batch * len(comm.p.windows_of[rank]) * comm.p.N


class _ShardedShiftExchangeAttnComm(_PortableAttnComm):
    """The routed exchange with token shards (SP > 1, any number of window groups, any owner map): rank ``(g, s)`` computes
    the query slots ``[s * shardN, (s + 1) * shardN)`` of the (shifted) windows its group owns. One all-to-all-v brings
    the q rows of those slots, another the k / v rows of all slots of those windows, each from the rank that holds the
    token - ``(owner of its window, its shard)`` -, and a third returns the outputs along the reversed q routes. For
    unshifted blocks the q rows are local and the k / v exchange stays inside the group."""

    def __init__(self, pctx: "ParallelContext", batch: int):
        super().__init__(pctx, batch)
        self._tables = {}

    def _rows_held(self, rank_index):
        p = self.p
        return self.batch * len(p.windows_of[rank_index // p.sp]) * p.shardN

    def _needs(self, rank_index, shifted, queries_only):
        """(source rank, source row) of every (batch, owned window, slot) the rank needs, in that order; slots are its
        query slots or all of them."""
        p, Bn, N, sN = self.p, self.batch, self.p.N, self.p.shardN
        g, s = divmod(rank_index, p.sp)
        src_win, src_tok, _ = self._sources[shifted]
        wins = np.asarray(p.windows_of[g])
        slots = np.arange(s * sN, (s + 1) * sN) if queries_only else np.arange(N)
        sw, st = src_win[wins][:, slots], src_tok[wins][:, slots]                          # [nW_g, slots]
        rank = self._owner[sw] * p.sp + st // sN
        held = self._counts[self._owner[sw]]                                               # windows held by the source rank
        row = (np.arange(Bn)[:, None, None] * held[None] + self._local_idx[sw][None]) * sN + (st % sN)[None]
        return np.broadcast_to(rank[None], row.shape).reshape(-1), row.reshape(-1)

    def _route(self, shifted, queries_only, device):
        p = self.p
        world = p.n_wg * p.sp
        me = p.wg_rank * p.sp + p.sp_rank
        rank, row = self._needs(me, shifted, queries_only)
        held = self._rows_held(me)
        recv_sizes = [int(((rank == r) & (r != me)).sum()) for r in range(world)]
        start = np.concatenate([[0], np.cumsum(recv_sizes)])
        assemble = np.empty(rank.shape[0], dtype=np.int64)
        assemble[rank == me] = row[rank == me]
        for r in range(world):
            if r != me and recv_sizes[r]:
                assemble[rank == r] = held + start[r] + np.arange(recv_sizes[r])
        send_index, send_sizes = [], []
        for d in range(world):
            if d == me:
                send_sizes.append(0)
                continue
            d_rank, d_row = self._needs(d, shifted, queries_only)
            pick = d_rank == me
            send_index.append(d_row[pick])
            send_sizes.append(int(pick.sum()))
        send_index = np.concatenate(send_index) if send_index else np.zeros(0, dtype=np.int64)
        out = dict(send_sizes=send_sizes, recv_sizes=recv_sizes)
        to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
        out.update(send_index=to(send_index), assemble=to(assemble))
        if queries_only:
            # the way back: what I received returns in the order it came; my home rows are rows I computed or rows of
            # the returned chunk, which arrives in my send order
            back = np.concatenate([np.nonzero(rank == r)[0] for r in range(world) if r != me] or [np.zeros(0, dtype=np.int64)])
            home = np.full(held, -1, dtype=np.int64)
            home[row[rank == me]] = np.nonzero(rank == me)[0]
            home[send_index] = rank.shape[0] + np.arange(send_index.shape[0])
            if (home < 0).any():
                raise RuntimeError("shift exchange: a home row has no producer (owner map and routes disagree)")
            out.update(return_index=to(back), home=to(home))
        return out

    def _tables_for(self, shifted, device):
        key = (bool(shifted), str(device))
        if key not in self._tables:
            p = self.p
            if not hasattr(self, "_sources"):
                gfull = WindowGeometry(self.batch, p.nWh, p.nWw, p.wh, p.ww)
                self._sources = {flag: tuple(t.numpy() for t in shifted_window_sources(gfull, flag)) for flag in (False, True)}
                self._owner = np.asarray(p.owner)
                self._counts = np.asarray([len(w) for w in p.windows_of])
                self._local_idx = np.zeros(self._owner.shape[0], dtype=np.int64)
                for g in range(p.n_wg):
                    self._local_idx[p.windows_of[g]] = np.arange(len(p.windows_of[g]))
            reg = self._sources[shifted][2][np.asarray(p.windows_of[p.wg_rank])]               # [nWl, N]
            self._tables[key] = dict(q=self._route(shifted, True, device), kv=self._route(shifted, False, device),
                                     reg=torch.from_numpy(np.ascontiguousarray(reg)).to(device),
                                     masked=bool((reg != reg[:, :1]).any()))
        return self._tables[key]

    def window_attention_portable(self, qkv, geo, num_heads, shifted, bias_table, use_mask, scale):
        from ..ops.attention import attention_core_reference, relative_position_index

        p, Bn, N, sN = self.p, self.batch, self.p.N, self.p.shardN
        Cd = qkv.shape[-1] // 3
        hd = Cd // num_heads
        nWl = len(p.windows_of[p.wg_rank])
        t = self._tables_for(shifted, qkv.device)
        group = p.manager.xfmr_tp_param_group

        def pull(cols, route):
            got = C.all_to_all_rows(cols.index_select(0, route["send_index"]), group, route["send_sizes"], route["recv_sizes"])
            return torch.cat([cols, got], 0).index_select(0, route["assemble"])

        q = pull(qkv[:, :Cd].contiguous(), t["q"]).reshape(Bn * nWl, sN, num_heads, hd).permute(0, 2, 1, 3)
        kv = pull(qkv[:, Cd:].contiguous(), t["kv"]).reshape(Bn * nWl, N, 2, num_heads, hd)
        k, v = kv[:, :, 0].permute(0, 2, 1, 3), kv[:, :, 1].permute(0, 2, 1, 3)
        mine = slice(p.sp_rank * sN, (p.sp_rank + 1) * sN)
        bias = None
        if bias_table is not None:
            idx = relative_position_index(p.wh, p.ww).to(bias_table.device)
            bias = bias_table[idx.reshape(-1)].reshape(N, N, num_heads).permute(2, 0, 1)[:, mine].to(q.dtype)
        mask = None
        if use_mask and shifted and t["masked"]:
            reg = t["reg"]
            mask = ((reg[:, mine, None] != reg[:, None, :]).to(q.dtype) * -100.0).repeat(Bn, 1, 1)
        o = attention_core_reference(q, k, v, scale, bias, mask).permute(0, 2, 1, 3).reshape(Bn * nWl * sN, Cd)
        route = t["q"]
        back = C.all_to_all_rows(o.index_select(0, route["return_index"]), group, route["recv_sizes"], route["send_sizes"])
        return torch.cat([o, back], 0).index_select(0, route["home"])


class _UlyssesAttnComm(_PortableAttnComm):
    """Sequence-parallel window attention by head <-> token all-to-all (DeepSpeed-Ulysses, the reference's
    ``WPUlyssesWindowAttention``: models/attention.py:795-819, 912-918; core/tensor_parallel.py:291-356): the token
    shards of all windows are exchanged for head groups, every rank runs ordinary single-rank window attention on all
    tokens of ``heads / sp`` heads, and a second all-to-all brings the outputs back to token shards. The collective
    baseline of the peer-memory K/V gather (``comm_backend: nccl`` and gloo ranks), used when one window group spans
    the set (``n_wg == 1``) and the local head count divides by ``sp``; otherwise the gather path of the base class
    runs. ``TERRA_SP_BASELINE=gather`` forces the latter."""

    def window_attention_portable(self, qkv, geo, num_heads, shifted, bias_table, use_mask, scale):
        p, m = self.p, self.p.manager
        sp, sN, N, Bn = p.sp, p.shardN, p.N, self.batch
        if num_heads % sp != 0 or p.n_wg != 1:
            return super().window_attention_portable(qkv, geo, num_heads, shifted, bias_table, use_mask, scale)
        group = m.xfmr_tp_param_group                  # the sp ranks that share this TP rank (n_wg == 1)
        nW = p.nWh * p.nWw
        rows = Bn * nW * sN
        Cl = qkv.shape[-1] // 3
        Cd, hd = Cl // sp, Cl // num_heads
        # head groups to their ranks: chunk d of the send buffer = (q | k | v) columns of head group d
        q, k, v = qkv.reshape(rows, 3, sp, Cd).unbind(1)
        send = torch.stack([q, k, v], dim=2).permute(1, 0, 2, 3).reshape(sp * rows, 3 * Cd)      # [d][row][q|k|v]
        recv = C.all_to_all_rows(send.contiguous(), group)                                      # [source shard][row][q|k|v]
        full = recv.reshape(sp, Bn, nW, sN, 3 * Cd).permute(1, 2, 0, 3, 4).reshape(Bn * nW * N, 3 * Cd)
        mine = p.sp_rank * (num_heads // sp)
        table = None if bias_table is None else bias_table[:, mine:mine + num_heads // sp]
        gfull = WindowGeometry(Bn, p.nWh, p.nWw, p.wh, p.ww)
        o = window_attention(full.contiguous(), gfull, num_heads // sp, shifted, table, use_mask, scale, None)
        # token shards back to their ranks; the received head groups are concatenated along the channels
        back = o.reshape(Bn, nW, sp, sN, Cd).permute(2, 0, 1, 3, 4).reshape(sp * rows, Cd)
        got = C.all_to_all_rows(back.contiguous(), group)                                       # [head group][row][Cd]
        assert hd * (num_heads // sp) == Cd
        return got.reshape(sp, rows, Cd).permute(1, 0, 2).reshape(rows, Cl)
