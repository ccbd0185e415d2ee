"""Sharded AdamW (ZeRO-1 style) over the flat parameter arena.

Role in the system is that of the reference's ``DistributedAdamW`` (optimizer/distributed_adamw.py:8-334):
gradients are summed over the replica group of each parameter class - ``full_param_replica_group`` (DP x WP) for
replicated parameters, ``xfmr_tp_param_replica_group`` (DP x window group x SP at fixed TP) for TP shards - divided
by the DP size, the owner applies AdamW with fp32 moments, and the new values reach every replica.

What differs is the granularity: the arena segment of each class is cut into equal contiguous ranges, one per
rank of the replica group, so the step is exactly reduce-scatter -> update of the owned range (fp32 master,
moments) -> all-gather of the working copy. On NVLink the three phases are one kernel over peer memory
(``terra_b200.parallel.nvlink``); elsewhere they are a reduce-scatter / all-reduce, the fused AdamW kernel (or
its PyTorch restatement on CPU) and an all-gather.

Moments exist only for the owned range. ``state_dict()`` therefore holds this rank's slice and is saved per rank
(``ckpt_layout: rank_local``), as the reference does for its owner-only states.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from .. import _ext
from ..utils.flat_params import ALIGN, ParamArena, get_arena


class _Shard:
    def __init__(self, label, group, rank, size, start, end):
        self.label, self.group, self.rank, self.size = label, group, rank, size
        self.start, self.end = start, end                        # arena range of the whole segment
        n = end - start
        per = (n + size - 1) // size
        per = (per + ALIGN - 1) // ALIGN * ALIGN
        self.per = per
        self.lo = min(end, start + rank * per)
        self.hi = min(end, self.lo + per)
        self.exp_avg = None
        self.exp_avg_sq = None


class DistributedAdamW(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, manager=None, model=None,
                 average_grad=True, process_group=None):
        params = [p for p in (q[1] if isinstance(q, tuple) else q for q in params) if p.requires_grad]
        if not params:
            raise ValueError("DistributedAdamW received no trainable parameters")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.manager = manager
        self.average_grad = average_grad
        self.global_step = 0
        self.step_count = 0
        self.arena: Optional[ParamArena] = get_arena(model) if model is not None else None
        if self.arena is None:
            if model is None:
                raise ValueError("DistributedAdamW needs the model (its parameters are sharded through the flat arena)")
            self.arena = ParamArena(model)
        self.shards: List[_Shard] = []
        for seg in self.arena.segments:
            group, rank, size = self._resolve_group(seg.label, process_group)
            self.shards.append(_Shard(seg.label, group, rank, size, seg.start, seg.end))
        self.fused = None     # peer-memory implementation (attached by terra_b200.parallel.nvlink)
        if self.arena.bf16 is not None and any(sh.size > 1 for sh in self.shards):
            # the step refreshes every replica's bf16 working copy but only the owner's fp32 master: kernels that read a
            # parameter in fp32 take the widened working copy instead (ops/packed.py)
            for p in self.arena.params:
                p.terra_master_sharded = True

    def _resolve_group(self, label, process_group):
        live = dist.is_available() and dist.is_initialized()
        if self.manager is not None and live:
            if label == "xfmr_tp_param_group":
                g = self.manager.xfmr_tp_param_replica_group
            elif label == "full":
                g = self.manager.full_param_replica_group
            else:
                raise ValueError(f"Unknown terra_grad_reduce_group: {label}")
            return g, dist.get_rank(g), dist.get_world_size(g)
        if live and process_group is not None:
            return process_group, dist.get_rank(process_group), dist.get_world_size(process_group)
        return None, 0, 1

    def _divisor(self) -> float:
        if not self.average_grad:
            return 1.0
        if self.manager is not None:
            return float(max(1, int(self.manager.get_dp_group_size())))
        return 1.0

    def zero_grad(self, set_to_none: bool = False):
        self.arena.zero_grad()

    # ------------------------------------------------------------------ the step
    @torch.no_grad()
    def step(self, closure=None, grad_scale: float = 1.0):
        loss = closure() if closure is not None else None
        self.step_count += 1
        g0 = self.param_groups[0]
        scale = grad_scale / self._divisor()
        if self.fused is not None:
            self.fused.step(self, g0, scale)
        else:
            for sh in self.shards:
                self.portable_shard_step(sh, g0, scale)
        if self.arena.master.is_cuda:
            from ..ops.conv import invalidate_packed_weights

            invalidate_packed_weights()      # operands packed from the bf16 working copy are stale now
        return loss

    def portable_shard_step(self, sh: "_Shard", g0, scale):
        """Collective version of one shard's step: reduce-scatter, update of the owned range, all-gather."""
        a = self.arena
        n_own = sh.hi - sh.lo
        if sh.size > 1:
            self._reduce_scatter(a.grad, sh)
        if sh.exp_avg is None:
            sh.exp_avg = torch.zeros(max(n_own, 1), dtype=torch.float32, device=a.master.device)
            sh.exp_avg_sq = torch.zeros_like(sh.exp_avg)
        if n_own > 0:
            self._update(a, sh, g0, scale)
        if sh.size > 1:
            self._all_gather(a, sh)

    def _reduce_scatter(self, grad, sh: _Shard):
        seg = grad[sh.start:sh.end]
        uniform = (sh.end - sh.start) == sh.per * sh.size
        if uniform and dist.get_backend(sh.group) == "nccl":
            dist.reduce_scatter_tensor(grad[sh.lo:sh.hi], seg, group=sh.group)
        else:
            dist.all_reduce(seg, group=sh.group)

    def _update(self, a: ParamArena, sh: _Shard, g0, scale):
        lo, hi = sh.lo, sh.hi
        b1, b2 = g0["betas"]
        if a.master.is_cuda:
            _ext.load().adamw_step(a.master[lo:hi], sh.exp_avg[:hi - lo], sh.exp_avg_sq[:hi - lo], a.grad[lo:hi],
                                   a.bf16[lo:hi] if a.bf16 is not None else None, g0["lr"], b1, b2, g0["eps"],
                                   g0["weight_decay"], self.step_count, scale)
            return
        g = a.grad[lo:hi] * scale
        p = a.master[lo:hi]
        p.mul_(1 - g0["lr"] * g0["weight_decay"])
        m, v = sh.exp_avg[:hi - lo], sh.exp_avg_sq[:hi - lo]
        m.mul_(b1).add_(g, alpha=1 - b1)
        v.mul_(b2).addcmul_(g, g, value=1 - b2)
        bc1, bc2 = 1 - b1 ** self.step_count, 1 - b2 ** self.step_count
        denom = v.sqrt().div_(math.sqrt(bc2)).add_(g0["eps"])
        p.addcdiv_(m, denom, value=-g0["lr"] / bc1)

    def _all_gather(self, a: ParamArena, sh: _Shard):
        """Every replica receives the updated values: the bf16 working copy on GPU (masters of foreign ranges are
        refreshed from it on demand), the fp32 masters on CPU."""
        buf = a.bf16 if (a.bf16 is not None) else a.master
        n = sh.end - sh.start
        padded = sh.per * sh.size
        if padded == n and dist.get_backend(sh.group) == "nccl":
            dist.all_gather_into_tensor(buf[sh.start:sh.end], buf[sh.lo:sh.hi], group=sh.group)
        else:
            mine = buf.new_zeros(sh.per)
            mine[:sh.hi - sh.lo] = buf[sh.lo:sh.hi]
            parts = [torch.empty_like(mine) for _ in range(sh.size)]
            dist.all_gather(parts, mine, group=sh.group)
            full = torch.cat(parts)[:n]
            buf[sh.start:sh.end] = full
        if a.bf16 is not None:
            self._masters_stale = True

    def sync_masters(self):
        """Bring the fp32 masters of ranges owned by other ranks up to date (from the gathered working copy)."""
        a = self.arena
        if a.bf16 is None or not getattr(self, "_masters_stale", False):
            return
        for sh in self.shards:
            if sh.size > 1:
                if sh.lo > sh.start:
                    a.master[sh.start:sh.lo] = a.bf16[sh.start:sh.lo].float()
                if sh.hi < sh.end:
                    a.master[sh.hi:sh.end] = a.bf16[sh.hi:sh.end].float()
        self._masters_stale = False

    # ------------------------------------------------------------------ checkpoint surface
    def state_dict(self):
        return {
            "step": self.step_count,
            "global_step": self.global_step,
            "param_groups": [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups],
            "shards": [dict(label=s.label, rank=s.rank, size=s.size, lo=s.lo - s.start, hi=s.hi - s.start,
                            exp_avg=None if s.exp_avg is None else s.exp_avg.cpu(),
                            exp_avg_sq=None if s.exp_avg_sq is None else s.exp_avg_sq.cpu()) for s in self.shards],
        }

    def full_state_dict(self):
        """Collective. The optimizer state in ``torch.optim.AdamW``'s per-parameter layout (``state[i] = {step, exp_avg,
        exp_avg_sq}`` with whole-parameter fp32 tensors on the CPU, ``i`` in ``model.parameters()`` order) - what the
        reference's ``DistributedAdamW`` keeps per owned parameter (optimizer/distributed_adamw.py:282-323). The moments
        of every shard are gathered from their owners, so the result does not depend on how the arena was cut and can be
        loaded into another layout (``load_state_dict`` accepts it) or into ``torch.optim.AdamW``."""
        a = self.arena
        dev = a.master.device
        m_full = torch.zeros(a.numel, dtype=torch.float32, device=dev)
        v_full = torch.zeros(a.numel, dtype=torch.float32, device=dev)
        for sh in self.shards:
            n_own = sh.hi - sh.lo
            if sh.exp_avg is not None and n_own > 0:
                m_full[sh.lo:sh.hi] = sh.exp_avg[:n_own]
                v_full[sh.lo:sh.hi] = sh.exp_avg_sq[:n_own]
            if sh.size > 1:
                # every element has exactly one owner in the group: a sum puts the pieces together
                dist.all_reduce(m_full[sh.start:sh.end], group=sh.group)
                dist.all_reduce(v_full[sh.start:sh.end], group=sh.group)
        state = {}
        for i, (p, off) in enumerate(zip(a.params, a.offsets)):
            n = p.numel()
            state[i] = {"step": torch.tensor(float(self.step_count)), "exp_avg": m_full[off:off + n].view(p.shape).cpu().clone(),
                        "exp_avg_sq": v_full[off:off + n].view(p.shape).cpu().clone()}
        groups = [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups]
        groups[0]["params"] = list(range(len(a.params)))
        return {"state": state, "param_groups": groups, "global_step": self.global_step}

    def _load_per_parameter(self, state):
        a = self.arena
        dev = a.master.device
        m_full = torch.zeros(a.numel, dtype=torch.float32, device=dev)
        v_full = torch.zeros(a.numel, dtype=torch.float32, device=dev)
        steps = []
        for i, (p, off) in enumerate(zip(a.params, a.offsets)):
            st = state["state"].get(i, state["state"].get(str(i)))
            if st is None:
                continue          # owner-only files of the reference hold a subset: missing moments start at zero
            n = p.numel()
            m_full[off:off + n] = st["exp_avg"].reshape(-1).to(dev, torch.float32)
            v_full[off:off + n] = st["exp_avg_sq"].reshape(-1).to(dev, torch.float32)
            steps.append(int(float(st["step"])))
        self.step_count = max(steps) if steps else 0
        self.global_step = int(state.get("global_step", self.global_step))
        for g, saved in zip(self.param_groups, state.get("param_groups", [])):
            g.update({k: v for k, v in saved.items() if k != "params"})
        for sh in self.shards:
            n_own = max(sh.hi - sh.lo, 1)
            sh.exp_avg = torch.zeros(n_own, dtype=torch.float32, device=dev)
            sh.exp_avg_sq = torch.zeros(n_own, dtype=torch.float32, device=dev)
            if sh.hi > sh.lo:
                sh.exp_avg[:sh.hi - sh.lo] = m_full[sh.lo:sh.hi]
                sh.exp_avg_sq[:sh.hi - sh.lo] = v_full[sh.lo:sh.hi]

    def load_state_dict(self, state):
        if "shards" not in state and "state" in state:
            return self._load_per_parameter(state)      # torch.optim.AdamW / reference per-parameter layout
        self.step_count = int(state["step"])
        self.global_step = int(state.get("global_step", 0))
        for g, saved in zip(self.param_groups, state["param_groups"]):
            g.update(saved)
        for s, saved in zip(self.shards, state["shards"]):
            if saved["label"] != s.label or saved["size"] != s.size or saved["rank"] != s.rank:
                raise ValueError("DistributedAdamW state was written for a different layout")
            dev = self.arena.master.device
            s.exp_avg = None if saved["exp_avg"] is None else saved["exp_avg"].to(dev)
            s.exp_avg_sq = None if saved["exp_avg_sq"] is None else saved["exp_avg_sq"].to(dev)
