"""Masked L1 / MSE loss: ``criterion(pred * mask, label)`` with mean reduction (reference:
core/runtime/run_one_step.py:3-26, utils.py:82-91).

On CUDA one kernel reads pred / label / mask once, accumulates the loss and writes the gradient with respect to
``pred`` already multiplied by ``post_scale / n``; the returned loss is ``post_scale * mean(...)`` and its
backward hands that gradient on (the upstream gradient is expected to be 1, as in ``loss.backward()``).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _ext

KINDS = {"L1": 0, "L2": 1, "MSE": 1}


class _MaskedLossFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pred, label, mask, kind, post_scale):
        ext = _ext.load()
        n = pred.numel()
        loss_sum = torch.zeros(1, device=pred.device, dtype=torch.float32)
        grad = torch.empty_like(pred)
        ext.masked_loss(pred, label, mask, kind, float(post_scale) / n, loss_sum, grad)
        ctx.save_for_backward(grad)
        return (loss_sum * (float(post_scale) / n)).reshape(())

    @staticmethod
    def backward(ctx, g):
        (grad,) = ctx.saved_tensors
        return grad, None, None, None, None


def masked_loss(pred, label, mask: Optional[torch.Tensor], loss_func: str = "L1", post_scale: float = 1.0):
    """``post_scale * mean(f(pred * mask - label))``; ``mask`` broadcasts over the batch dimension."""
    kind = KINDS[loss_func]
    if pred.is_cuda:
        label = label.to(torch.bfloat16).contiguous()
        m = None if mask is None else mask.to(torch.bfloat16).contiguous()
        return _MaskedLossFn.apply(pred.contiguous(), label, m, kind, post_scale)
    out = pred if mask is None else pred * mask
    d = out - label
    loss = d.abs().mean() if kind == 0 else (d * d).mean()
    return loss.float() * post_scale
