"""Per-parameter cache of operands derived from the bf16 working copy (packed convolution weights, widened tables).

The reference has no counterpart: it hands ``nn.Conv2d`` / ``nn.Linear`` weights to cuDNN / cuBLAS as they are
(models/utils.py:101-177); here the implicit-GEMM kernels want tap-major packed weights, which are built once per
optimizer step instead of once per call.
"""
from __future__ import annotations

import torch

# Packed operands are functions of the bf16 working copy of a weight, which changes once per optimizer step. They are
# cached per parameter and rebuilt when the parameter's version counter (bumped by the in-place optimizer update of the
# master, or by a checkpoint load) or the working copy's address (arena rebinding) has moved.
_PACK_CACHE = {}


def _packed(weight, w16, kind, builder):
    import weakref

    key = (id(weight), kind)
    stamp = (weight._version, w16.data_ptr(), PACK_EPOCH[0])
    hit = _PACK_CACHE.get(key)
    if hit is not None and hit[0] == stamp and hit[2]() is weight:
        return hit[1]
    val = builder(w16)
    _PACK_CACHE[key] = (stamp, val, weakref.ref(weight))
    return val


def fp32_values(p):
    """The fp32 values of a parameter for a kernel that reads it in fp32 (the relative-position bias table). Under an
    optimizer that shards the fp32 masters only the owner's master is current, while the bf16 working copy is gathered
    to every rank after each step: there every rank, the owner included, reads the same widened copy of the working
    copy, rebuilt once per optimizer step. Otherwise the master itself."""
    if getattr(p, "bf16", None) is None or not getattr(p, "terra_master_sharded", False):
        return p.data
    return _packed(p, p.bf16, "f32", lambda t: t.float())


class _WidenedValues(torch.autograd.Function):
    """fp32 values of a parameter taken from its bf16 working copy; the gradient goes to the parameter unchanged."""

    @staticmethod
    def forward(ctx, p):
        return fp32_values(p).clone()

    @staticmethod
    def backward(ctx, g):
        return g


def fp32_param(p):
    """``p`` for differentiable PyTorch code that reads it in fp32 (the composed attention paths index the bias table):
    the parameter itself, unless its fp32 master is owner-only (or released, with sharded parameters) - then the widened
    working copy, with the gradient passed on to the parameter."""
    if getattr(p, "bf16", None) is None or not getattr(p, "terra_master_sharded", False):
        return p
    return _WidenedValues.apply(p)


PACK_EPOCH = [0]      # bumped by the optimizers after every step (the fused kernels write the working copy directly)


def invalidate_packed_weights() -> None:
    PACK_EPOCH[0] += 1
