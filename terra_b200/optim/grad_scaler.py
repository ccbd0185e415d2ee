"""Dynamic loss scaling for ``precision: fp16`` runs (reference: the ``torch.cuda.amp.GradScaler`` use of
core/runtime/run_model.py:424-448, 471-472, 512-514, 571-593).

The sm_100a kernels compute in bf16 whatever ``precision`` says (same tensor-core rate as fp16, wider exponent), so
overflow protection is not needed for the arithmetic; the scaler exists so that ``fp16`` configs keep their training
semantics: the loss gradient is multiplied by the scale, gradients are inspected for inf / nan in ONE pass over the
flat gradient arena (``grad_inspect`` kernel, which also yields the squared norm for clipping), the un-scaling (and the
clip coefficient) rides in the optimizer kernel's ``grad_scale``, a step with non-finite gradients is skipped on every
rank alike and the scale is backed off, and it grows again after ``growth_interval`` clean steps.
``state_dict()`` uses ``torch.amp.GradScaler``'s keys, so checkpoints are interchangeable.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


class LossScaler:
    def __init__(self, init_scale: float = 65536.0, growth_factor: float = 2.0, backoff_factor: float = 0.5,
                 growth_interval: int = 2000, enabled: bool = True):
        self._scale = float(init_scale)
        self.growth_factor, self.backoff_factor = float(growth_factor), float(backoff_factor)
        self.growth_interval = int(growth_interval)
        self._growth_tracker = 0
        self.enabled = enabled
        self.skipped_steps = 0
        self._buf: Optional[torch.Tensor] = None

    def get_scale(self) -> float:
        return self._scale if self.enabled else 1.0

    def is_enabled(self) -> bool:
        return self.enabled

    # ------------------------------------------------------------------ inspection
    def inspect(self, grad: torch.Tensor, group=None) -> Tuple[bool, float]:
        """``(found_inf, norm of grad / scale)`` over a flat fp32 gradient buffer; with ``group`` the inf flag is
        shared (any rank's overflow skips the step everywhere) while the norm stays this rank's own, as in the
        reference, whose ``clip_grad_norm_`` sees each rank's local gradients. Synchronises the host."""
        if grad.is_cuda:
            from .. import _ext

            if self._buf is None or self._buf.device != grad.device:
                self._buf = torch.zeros(2, dtype=torch.float32, device=grad.device)
            self._buf.zero_()
            _ext.load().grad_inspect(grad, self._buf)
            out = self._buf
        else:
            finite = torch.isfinite(grad).all()
            out = torch.stack([(grad.double() ** 2).sum().float() if finite else torch.zeros(()), (~finite).float()])
        if group is not None and dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            flag = out[1:2].clone()
            dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)
            sumsq, bad = float(out[0].item()), float(flag.item())
        else:
            sumsq, bad = (float(v) for v in out.tolist())
        return bad != 0.0, (sumsq ** 0.5) / self.get_scale()

    # ------------------------------------------------------------------ the step
    def step(self, optimizer, grad: torch.Tensor, clip_max_norm: Optional[float] = None, group=None) -> bool:
        """Inspect, then either run ``optimizer.step(grad_scale=...)`` with the un-scaling and the clip coefficient
        folded in, or skip. Returns ``True`` when the step ran. Call ``update()`` afterwards."""
        found_inf, norm = self.inspect(grad, group)
        return self.step_with_stats(optimizer, found_inf, norm * self.get_scale(), clip_max_norm)

    def step_with_stats(self, optimizer, found_inf: bool, scaled_norm: float, clip_max_norm: Optional[float] = None) -> bool:
        """The decision of ``step`` from statistics gathered elsewhere: ``scaled_norm`` is the norm of the gradients as
        they are (still multiplied by the loss scale)."""
        norm = scaled_norm / self.get_scale()
        self._found_inf = found_inf
        if found_inf:
            self.skipped_steps += 1
            return False
        coef = 1.0 / self.get_scale()
        if clip_max_norm is not None and norm > clip_max_norm:
            coef *= clip_max_norm / (norm + 1e-6)
        optimizer.step(grad_scale=coef)
        return True

    def update(self, found_inf: Optional[bool] = None) -> None:
        if not self.enabled:
            return
        bad = self._found_inf if found_inf is None else found_inf
        if bad:
            self._scale *= self.backoff_factor
            self._growth_tracker = 0
        else:
            self._growth_tracker += 1
            if self._growth_tracker >= self.growth_interval:
                self._scale *= self.growth_factor
                self._growth_tracker = 0

    # ------------------------------------------------------------------ checkpoint surface (torch.amp.GradScaler's keys)
    def state_dict(self):
        return {"scale": self._scale, "growth_factor": self.growth_factor, "backoff_factor": self.backoff_factor,
                "growth_interval": self.growth_interval, "_growth_tracker": self._growth_tracker}

    def load_state_dict(self, sd):
        self._scale = float(sd["scale"])
        self.growth_factor = float(sd.get("growth_factor", self.growth_factor))
        self.backoff_factor = float(sd.get("backoff_factor", self.backoff_factor))
        self.growth_interval = int(sd.get("growth_interval", self.growth_interval))
        self._growth_tracker = int(sd.get("_growth_tracker", 0))
