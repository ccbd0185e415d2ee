"""AdamW over a flat parameter arena: one kernel per step updates fp32 masters, both moments and the bf16
working copy. Hyper-parameters and update order follow the reference (optimizer/utils.py:8-98,
optimizer/distributed_adamw.py:305-323): decoupled decay first, bias-corrected moments, eps outside the root.

Without an arena (CPU, or a model that was not flattened) it defers to ``torch.optim.AdamW`` maths per parameter.
"""
from __future__ import annotations

import math

import torch

from .. import _ext
from ..utils.flat_params import get_arena


def _invalidate_packed():
    from ..ops.conv import invalidate_packed_weights

    invalidate_packed_weights()


class FusedAdamW(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, model=None):
        params = list(params)
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.arena = get_arena(model) if model is not None else None
        self.global_step = 0
        self._flat = None

    def _flat_state(self):
        if self._flat is None:
            a = self.arena
            self._flat = dict(step=0, exp_avg=torch.zeros_like(a.master), exp_avg_sq=torch.zeros_like(a.master))
        return self._flat

    def zero_grad(self, set_to_none: bool = False):
        if self.arena is not None:
            self.arena.zero_grad()
        else:
            super().zero_grad(set_to_none=set_to_none)

    @torch.no_grad()
    def step(self, closure=None, grad_scale: float = 1.0):
        loss = closure() if closure is not None else None
        g0 = self.param_groups[0]
        if self.arena is not None and self.arena.master.is_cuda and len(self.param_groups) == 1:
            st = self._flat_state()
            st["step"] += 1
            a = self.arena
            _ext.load().adamw_step(a.master, st["exp_avg"], st["exp_avg_sq"], a.grad, a.bf16, g0["lr"], g0["betas"][0],
                                   g0["betas"][1], g0["eps"], g0["weight_decay"], st["step"], grad_scale)
            _invalidate_packed()
            return loss
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                st["step"] += 1
                g = p.grad.float() * grad_scale
                pf = p.data.float()
                pf.mul_(1 - group["lr"] * group["weight_decay"])
                st["exp_avg"].mul_(b1).add_(g, alpha=1 - b1)
                st["exp_avg_sq"].mul_(b2).addcmul_(g, g, value=1 - b2)
                bc1 = 1 - b1 ** st["step"]
                bc2 = 1 - b2 ** st["step"]
                denom = st["exp_avg_sq"].sqrt().div_(math.sqrt(bc2)).add_(group["eps"])
                pf.addcdiv_(st["exp_avg"], denom, value=-group["lr"] / bc1)
                p.data.copy_(pf)
        if self.arena is not None:
            self.arena.sync_bf16()
        return loss

    # ---- per-parameter view of the flat state, so that checkpoints look like torch.optim.AdamW's
    def state_dict(self):
        if self._flat is not None and self.arena is not None:
            for p, off in zip(self.arena.params, self.arena.offsets):
                n = p.numel()
                self.state[p] = dict(step=self._flat["step"],
                                     exp_avg=self._flat["exp_avg"][off:off + n].view(p.shape),
                                     exp_avg_sq=self._flat["exp_avg_sq"][off:off + n].view(p.shape))
        return super().state_dict()

    def load_state_dict(self, state_dict):
        super().load_state_dict(state_dict)
        if self.arena is not None and self.arena.master.is_cuda:
            st = self._flat_state()
            for p, off in zip(self.arena.params, self.arena.offsets):
                s = self.state.get(p)
                if s:
                    n = p.numel()
                    st["exp_avg"][off:off + n].copy_(s["exp_avg"].reshape(-1))
                    st["exp_avg_sq"][off:off + n].copy_(s["exp_avg_sq"].reshape(-1))
                    st["step"] = int(s["step"])
