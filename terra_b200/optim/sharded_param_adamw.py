"""AdamW over sharded parameters (the optimizer half of ``terra_b200.parallel.param_sharding``).

Under the reference's FSDP configurations (``optimizer_config`` 5, 7, 8, 9) a plain ``torch.optim.AdamW`` runs on each
rank's flat parameter shards, whose gradients FSDP has reduce-scattered (models/model_utils/get_model.py:1196-1283,
optimizer/utils.py). Here the shards are the owned slices of the units' arenas: ``step`` first lets the sharder finish the
backward pass (reduce-scatter of what is still resident), then updates every owned slice - fp32 values, fp32 moments, and
on the GPU the owned bf16 slice the next all-gather reads - with the same fused kernel as the other optimizers. Nothing is
gathered after the step: the next forward pass does that unit by unit.

The gradient convention is the sharded optimizer's (``DistributedAdamW``): sums over each label's replica group, divided
by the data-parallel size.
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch
import torch.distributed as dist

from .. import _ext
from ..parallel.param_sharding import ParamSharder


class ShardedParamAdamW(torch.optim.Optimizer):
    def __init__(self, sharder: ParamSharder, lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, manager=None,
                 average_grad=True):
        self.sharder = sharder
        # the parameter group lists the owned slices, which are what this rank optimises
        slices = [r.own_master for u in sharder.all_units() for r in u.ranges]
        super().__init__(slices, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.manager = manager
        self.average_grad = average_grad
        self.global_step = 0
        self.step_count = 0

    def _divisor(self) -> float:
        if self.average_grad and self.manager is not None:
            return float(max(1, int(self.manager.get_dp_group_size())))
        return 1.0

    def zero_grad(self, set_to_none: bool = False):
        self.sharder.zero_grad()

    def _ranges(self):
        for u in self.sharder.all_units():
            for r in u.ranges:
                yield u, r

    # ------------------------------------------------------------------ gradient statistics (clipping, loss scaling)
    @torch.no_grad()
    def gradient_stats(self):
        """Collective. ``(found_inf, norm)`` of the reduced gradient as this rank's model sees it: each label's owned
        slices are summed over the label's group, so every rank of a replica group gets the same value."""
        self.sharder.finish_backward()
        total, bad = None, None
        per_group: Dict[int, list] = {}
        for _, r in self._ranges():
            sq = (r.own_grad.double() ** 2).sum()
            finite = torch.isfinite(r.own_grad).all()
            ent = per_group.setdefault(id(r.group), [r.group, r.size, torch.zeros((), dtype=torch.float64, device=sq.device),
                                                     torch.zeros((), dtype=torch.float64, device=sq.device)])
            ent[2] += torch.where(finite, sq, torch.zeros_like(sq))
            ent[3] += (~finite).double()
        for group, size, sq, nonfinite in per_group.values():
            both = torch.stack([sq, nonfinite])
            if size > 1:
                dist.all_reduce(both, group=group)
            total = both[0] if total is None else total + both[0]
            bad = both[1] if bad is None else bad + both[1]
        if dist.is_available() and dist.is_initialized():
            flag = bad.clone()
            dist.all_reduce(flag, op=dist.ReduceOp.MAX)       # a non-finite gradient anywhere skips the step everywhere
            bad = flag
        return bool(bad.item() != 0), float(total.sqrt().item())

    @torch.no_grad()
    def clip_grad_norm_(self, max_norm: float) -> float:
        found_inf, norm = self.gradient_stats()
        if norm > max_norm:
            coef = max_norm / (norm + 1e-6)
            for _, r in self._ranges():
                r.own_grad.mul_(coef)
        return norm

    # ------------------------------------------------------------------ the step
    @torch.no_grad()
    def step(self, closure=None, grad_scale: float = 1.0):
        loss = closure() if closure is not None else None
        self.sharder.finish_backward()
        self.step_count += 1
        g0 = self.param_groups[0]
        scale = grad_scale / self._divisor()
        b1, b2 = g0["betas"]
        for u, r in self._ranges():
            if r.exp_avg is None:
                r.exp_avg = torch.zeros_like(r.own_master)
                r.exp_avg_sq = torch.zeros_like(r.own_master)
            if r.own_master.is_cuda:
                _ext.load().adamw_step(r.own_master, r.exp_avg, r.exp_avg_sq, r.own_grad, r.own_work, g0["lr"], b1, b2,
                                       g0["eps"], g0["weight_decay"], self.step_count, scale)
                continue
            g = r.own_grad * scale
            r.own_master.mul_(1 - g0["lr"] * g0["weight_decay"])
            r.exp_avg.mul_(b1).add_(g, alpha=1 - b1)
            r.exp_avg_sq.mul_(b2).addcmul_(g, g, value=1 - b2)
            bc1, bc2 = 1 - b1 ** self.step_count, 1 - b2 ** self.step_count
            denom = r.exp_avg_sq.sqrt().div_(math.sqrt(bc2)).add_(g0["eps"])
            r.own_master.addcdiv_(r.exp_avg, denom, value=-g0["lr"] / bc1)
            if r.own_work is not None:
                r.own_work.copy_(r.own_master)           # the kernel writes the bf16 slice itself
        return loss

    # ------------------------------------------------------------------ checkpoint surface
    def _groups_without_params(self) -> List[dict]:
        return [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups]

    def state_dict(self):
        """This rank's slices (saved per rank, ``fsdp_checkpoint_type: sharded``)."""
        return {
            "step": self.step_count, "global_step": self.global_step, "param_groups": self._groups_without_params(),
            "unit_shards": [dict(unit=u.name, label=r.label, rank=r.rank, size=r.size, lo=r.lo, hi=r.hi,
                                 exp_avg=None if r.exp_avg is None else r.exp_avg.cpu(),
                                 exp_avg_sq=None if r.exp_avg_sq is None else r.exp_avg_sq.cpu())
                            for u, r in self._ranges()],
        }

    def _gather_flat(self, u, pick) -> torch.Tensor:
        """A unit-long fp32 tensor put together from every owner's slice (``pick(range)`` or zeros)."""
        full = torch.zeros(u.arena.numel, dtype=torch.float32, device=u.ranges[0].own_master.device)
        for r in u.ranges:
            mine = pick(r)
            mine = torch.zeros_like(r.own_master) if mine is None else mine
            if r.size > 1:
                dist.all_gather_into_tensor(full[r.start:r.end], mine, group=r.group)
            else:
                full[r.start:r.end].copy_(mine)
        return full

    @torch.no_grad()
    def full_state_dict(self):
        """Collective. ``torch.optim.AdamW``'s layout: ``state[i] = {step, exp_avg, exp_avg_sq}`` with whole-parameter
        fp32 CPU tensors, ``i`` in ``model.parameters()`` order (``fsdp_checkpoint_type: full``; what FSDP's full optimizer
        state dict gives the reference, train_scripts/train.py:130-213). Independent of how the units were cut."""
        index = {id(p): i for i, p in enumerate(self.sharder.param_order)}
        state = {}
        for u in self.sharder.all_units():
            m = self._gather_flat(u, lambda r: r.exp_avg)
            v = self._gather_flat(u, lambda r: r.exp_avg_sq)
            for p, off in zip(u.arena.params, u.arena.offsets):
                n = p.numel()
                state[index[id(p)]] = {"step": torch.tensor(float(self.step_count)),
                                       "exp_avg": m[off:off + n].view(p.shape).cpu().clone(),
                                       "exp_avg_sq": v[off:off + n].view(p.shape).cpu().clone()}
        groups = self._groups_without_params()
        groups[0]["params"] = list(range(len(self.sharder.param_order)))
        return {"state": dict(sorted(state.items())), "param_groups": groups, "global_step": self.global_step}

    def _load_hyperparameters(self, saved_groups):
        for g, saved in zip(self.param_groups, saved_groups or []):
            g.update({k: v for k, v in saved.items() if k != "params"})

    @torch.no_grad()
    def load_state_dict(self, state):
        if "unit_shards" in state:
            self.step_count = int(state["step"])
            self.global_step = int(state.get("global_step", 0))
            self._load_hyperparameters(state.get("param_groups"))
            saved = state["unit_shards"]
            mine = list(self._ranges())
            if len(saved) != len(mine):
                raise ValueError("sharded optimizer state was written for a different unit layout")
            for (u, r), s in zip(mine, saved):
                if (s["unit"], s["label"], s["rank"], s["size"], s["lo"], s["hi"]) != (u.name, r.label, r.rank, r.size, r.lo, r.hi):
                    raise ValueError("sharded optimizer state was written for a different layout (use "
                                     "fsdp_checkpoint_type: full to move between layouts)")
                dev = r.own_master.device
                r.exp_avg = None if s["exp_avg"] is None else s["exp_avg"].to(dev)
                r.exp_avg_sq = None if s["exp_avg_sq"] is None else s["exp_avg_sq"].to(dev)
            return
        if "state" not in state:
            raise ValueError("unrecognised optimizer state: neither this optimizer's shards nor a per-parameter state")
        # per-parameter layout (torch.optim.AdamW, the sharded optimizer's full_state_dict, the reference's files)
        index = {id(p): i for i, p in enumerate(self.sharder.param_order)}
        steps = []
        for u in self.sharder.all_units():
            dev = u.ranges[0].own_master.device
            m = torch.zeros(u.arena.numel, dtype=torch.float32, device=dev)
            v = torch.zeros_like(m)
            for p, off in zip(u.arena.params, u.arena.offsets):
                i = index[id(p)]
                st = state["state"].get(i, state["state"].get(str(i)))
                if st is None:
                    continue
                n = p.numel()
                m[off:off + n] = st["exp_avg"].reshape(-1).to(dev, torch.float32)
                v[off:off + n] = st["exp_avg_sq"].reshape(-1).to(dev, torch.float32)
                steps.append(int(float(st["step"])))
            for r in u.ranges:
                r.exp_avg = m[r.lo:r.hi].clone()
                r.exp_avg_sq = v[r.lo:r.hi].clone()
        self.step_count = max(steps) if steps else 0
        self.global_step = int(state.get("global_step", self.global_step))
        self._load_hyperparameters(state.get("param_groups"))
