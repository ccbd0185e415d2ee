"""Generic domain (row-stripe) parallelism for convolutional models: a tensor is cut along one spatial dimension over
the ranks of a group, and the layers whose receptive field or statistics cross the cut get what they need from the
neighbours.

    dom = DomainGroup(group)                          # or DomainGroup(manager=parallel_manager)
    model = convert_to_domain_parallel(model, dom)    # Conv2d/3d, ConvTranspose2d/3d, GroupNorm replaced in place
    y_local = model(shard_tensor(x, -2, dom))
    y = gather_tensor(y_local, -2, dom)

Capabilities of the reference's ``credit/domain_parallel`` package (sharding.py:11-107, halo_exchange.py:18-205,
layers.py:87-580, convert.py:76-240), built on this repository's autograd-aware collectives, so every layer is
differentiable and runs on gloo CPU ranks as well as on NCCL:

* ``HaloExchange``: rows from both neighbours in front of and behind the local rows (zeros at the ends of the domain),
  gradients of the halo rows travel back and are added where the rows came from;
* convolutions: the padding along the cut dimension becomes halo rows, the layer then runs unpadded in that dimension;
  transposed convolutions with overlapping outputs exchange *input* rows, compute the overlap locally and trim it;
* ``DomainParallelGroupNorm``: the per-(sample, group) sums are all-reduced, so the statistics are those of the whole
  domain;
* ``DomainParallelPeriodicConv2d`` (circular in W, halo in H) and ``DomainParallelInterpolate``.

The model of this repository does not go through these generic wrappers: its down / up-sampling blocks call the fused
sm_100a kernels with the halo rows pushed over NVLink (``ops/conv.py``, ``parallel/nvlink.py::PeerDomain``). This module
is for other convolutional stacks that want the same decomposition.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from . import collectives as C


class DomainGroup:
    """Where this rank sits in the decomposition: ``size`` ranks in group order, stripe ``rank``, and the global ranks of
    the neighbours (``None`` at the ends). Built from a process group, or from a ``ParallelManager`` (its
    window-parallel group is the domain group of the convolution stage)."""

    def __init__(self, group=None, manager=None):
        if group is None and manager is not None:
            group = manager.window_parallel_group
        self.group = group
        live = dist.is_available() and dist.is_initialized()
        self.size = dist.get_world_size(group) if live else 1
        self.rank = dist.get_rank(group) if live else 0
        to_global = (lambda r: dist.get_global_rank(group, r)) if (live and group is not None) else (lambda r: r)
        self.prev = to_global(self.rank - 1) if self.rank > 0 else None
        self.next = to_global(self.rank + 1) if self.rank < self.size - 1 else None

    @property
    def active(self) -> bool:
        return self.size > 1


def _dom(dom) -> DomainGroup:
    if isinstance(dom, DomainGroup):
        return dom
    if dom is None:
        return DomainGroup()
    if hasattr(dom, "window_parallel_group"):
        return DomainGroup(manager=dom)
    return DomainGroup(group=dom)


# ------------------------------------------------------------------------------------------------ sharding
def shard_tensor(x: torch.Tensor, dim: int = -2, dom=None) -> torch.Tensor:
    """This rank's equal share of ``x`` along ``dim``."""
    d = _dom(dom)
    if not d.active:
        return x
    dim = dim % x.ndim
    if x.shape[dim] % d.size:
        raise ValueError(f"Cannot shard dim {dim} of size {x.shape[dim]} evenly across {d.size} domain-parallel ranks")
    per = x.shape[dim] // d.size
    return x.narrow(dim, d.rank * per, per).contiguous()


def gather_tensor(x: torch.Tensor, dim: int = -2, dom=None) -> torch.Tensor:
    """Concatenation of every rank's shard along ``dim`` (differentiable: the gradient of a gathered tensor is
    reduce-scattered back to the shards)."""
    d = _dom(dom)
    if not d.active:
        return x
    dim = dim % x.ndim
    return C.all_gather_rows(x.movedim(dim, 0).contiguous(), d.group).movedim(0, dim).contiguous()


def shard_batch(batch: dict, spatial_dims_5d: int = -2, spatial_dims_4d: int = -2, dom=None) -> dict:
    """Shard every 4-D ``[B, C, H, W]`` and 5-D ``[B, C, T, H, W]`` tensor of a batch dictionary; other entries pass."""
    d = _dom(dom)
    if not d.active:
        return batch
    out = {}
    for key, val in batch.items():
        if isinstance(val, torch.Tensor) and val.ndim == 5:
            out[key] = shard_tensor(val, spatial_dims_5d, d)
        elif isinstance(val, torch.Tensor) and val.ndim == 4:
            out[key] = shard_tensor(val, spatial_dims_4d, d)
        else:
            out[key] = val
    return out


# ------------------------------------------------------------------------------------------------ halo exchange
class HaloExchange(nn.Module):
    """``halo_width`` rows of each neighbour attached in front of and behind the local rows along ``dim``."""

    def __init__(self, halo_width: int, dim: int = -2, dom=None):
        super().__init__()
        self.halo_width, self.dim, self.dom = int(halo_width), dim, _dom(dom)

    def forward(self, x):
        d = self.dom
        if self.halo_width <= 0 or not d.active:
            return x
        dim = self.dim % x.ndim
        if x.shape[dim] < self.halo_width:
            raise ValueError(f"local extent {x.shape[dim]} is smaller than the halo width {self.halo_width}")
        moved = x.movedim(dim, 2) if dim != 2 else x
        out = C.halo_rows(moved.contiguous(), self.halo_width, d.prev, d.next, d.group)
        return out.movedim(2, dim) if dim != 2 else out

    @staticmethod
    def trim(x, halo_before: int, halo_after: int, dim: int = -2):
        dim = dim % x.ndim
        return x.narrow(dim, halo_before, x.shape[dim] - halo_before - halo_after)


def _component(v, index):
    return v if isinstance(v, int) else v[index]


def _without(padding, index, rank):
    """The padding tuple with the cut dimension's entry set to zero."""
    full = [padding] * rank if isinstance(padding, int) else list(padding)
    full[index] = 0
    return tuple(full)


class _DomainParallelConvNd(nn.Module):
    """Convolution (2-D or 3-D) whose padding along the cut dimension is supplied by the neighbours."""

    RANK = 2

    def __init__(self, conv, shard_dim: int, dom=None):
        super().__init__()
        self.conv, self.shard_dim, self.dom = conv, shard_dim, _dom(dom)
        self.axis = (shard_dim % (self.RANK + 2)) - 2               # index of the cut dimension in kernel_size etc.
        if isinstance(conv.padding, str):
            raise NotImplementedError("string paddings ('same', 'valid') are not supported by the domain-parallel wrapper")
        k, s = _component(conv.kernel_size, self.axis), _component(conv.stride, self.axis)
        p, dl = _component(conv.padding, self.axis), _component(conv.dilation, self.axis)
        self.halo_width = p
        self.effective_kernel = dl * (k - 1) + 1
        self.stride_h = s
        self.halo = HaloExchange(p, shard_dim, self.dom)

    def _op(self, x, padding):
        fn = F.conv2d if self.RANK == 2 else F.conv3d
        return fn(x, self.conv.weight, self.conv.bias, self.conv.stride, padding, self.conv.dilation, self.conv.groups)

    def forward(self, x):
        if not self.dom.active:
            return self.conv(x)
        if self.halo_width == 0:
            if self.effective_kernel > self.stride_h:
                raise NotImplementedError("a convolution without padding whose receptive fields overlap along the cut "
                                          "dimension needs output-range-aware sharding, which this wrapper does not do")
            return self.conv(x)
        return self._op(self.halo(x), _without(self.conv.padding, self.axis, self.RANK))

    @property
    def weight(self):
        return self.conv.weight

    @property
    def bias(self):
        return self.conv.bias


class DomainParallelConv2d(_DomainParallelConvNd):
    """``nn.Conv2d`` on a tensor cut along ``shard_dim`` (``-2``: H of ``[B, C, H, W]``)."""

    RANK = 2

    def __init__(self, conv: nn.Conv2d, shard_dim: int = -2, dom=None):
        super().__init__(conv, shard_dim, dom)


class DomainParallelConv3d(_DomainParallelConvNd):
    """``nn.Conv3d`` on ``[B, C, T, H, W]`` cut along ``shard_dim`` (``3``: H)."""

    RANK = 3

    def __init__(self, conv: nn.Conv3d, shard_dim: int = 3, dom=None):
        super().__init__(conv, shard_dim, dom)


class _DomainParallelConvTransposeNd(nn.Module):
    """Transposed convolution. Kernel <= stride along the cut: purely local. Otherwise neighbouring outputs overlap:
    ``padding`` input rows of each neighbour are attached, the layer runs without padding along the cut, and the rows
    that belong to the neighbours (each halo row yields ``stride`` rows, the dropped padding ``padding`` more) are
    trimmed."""

    RANK = 2

    def __init__(self, conv, shard_dim: int, dom=None):
        super().__init__()
        self.conv, self.shard_dim, self.dom = conv, shard_dim, _dom(dom)
        self.axis = (shard_dim % (self.RANK + 2)) - 2
        k, s = _component(conv.kernel_size, self.axis), _component(conv.stride, self.axis)
        p = _component(conv.padding, self.axis)
        self.stride_h = s
        self.halo_width = p if k > s else 0
        self.halo = HaloExchange(self.halo_width, shard_dim, self.dom)

    def forward(self, x):
        if not self.dom.active or self.halo_width == 0:
            return self.conv(x)
        fn = F.conv_transpose2d if self.RANK == 2 else F.conv_transpose3d
        out = fn(self.halo(x), self.conv.weight, self.conv.bias, self.conv.stride,
                 _without(self.conv.padding, self.axis, self.RANK), self.conv.output_padding, self.conv.groups,
                 self.conv.dilation)
        cut = self.halo_width * (self.stride_h + 1)
        return HaloExchange.trim(out, cut, cut, self.shard_dim % out.ndim)

    @property
    def weight(self):
        return self.conv.weight

    @property
    def bias(self):
        return self.conv.bias


class DomainParallelConvTranspose2d(_DomainParallelConvTransposeNd):
    RANK = 2

    def __init__(self, conv: nn.ConvTranspose2d, shard_dim: int = -2, dom=None):
        super().__init__(conv, shard_dim, dom)


class DomainParallelConvTranspose3d(_DomainParallelConvTransposeNd):
    RANK = 3

    def __init__(self, conv: nn.ConvTranspose3d, shard_dim: int = 3, dom=None):
        super().__init__(conv, shard_dim, dom)


class DomainParallelGroupNorm(nn.Module):
    """``nn.GroupNorm`` with the statistics of the whole domain: the per-(sample, group) sum and sum of squares are
    all-reduced over the group (one small collective forward, its adjoint backward)."""

    def __init__(self, norm: nn.GroupNorm, dom=None):
        super().__init__()
        self.num_groups, self.num_channels, self.eps, self.affine = norm.num_groups, norm.num_channels, norm.eps, norm.affine
        if self.affine:
            self.weight, self.bias = norm.weight, norm.bias
        else:
            self.register_parameter("weight", None)
            self.register_parameter("bias", None)
        self.dom = _dom(dom)

    def forward(self, x):
        d = self.dom
        if not d.active:
            return F.group_norm(x, self.num_groups, self.weight, self.bias, self.eps)
        B, Cn = x.shape[:2]
        xg = x.reshape(B, self.num_groups, -1)
        sums = torch.stack([xg.sum(-1), (xg * xg).sum(-1)], dim=-1)                  # [B, G, 2]
        sums = C.all_reduce_sum(sums, d.group)
        count = xg.shape[-1] * d.size
        mean = sums[..., 0] / count
        var = (sums[..., 1] / count - mean * mean).clamp_min(0.0)
        y = ((xg - mean[..., None]) * torch.rsqrt(var[..., None] + self.eps)).reshape(x.shape)
        if self.affine:
            shape = [1, Cn] + [1] * (x.ndim - 2)
            y = y * self.weight.view(shape) + self.bias.view(shape)
        return y


class DomainParallelPeriodicConv2d(nn.Module):
    """A convolution that pads W circularly (longitude) and H by reflection before an unpadded ``nn.Conv2d``
    (``periodic_conv.conv``, ``periodic_conv.padding``): with H cut over ranks the H padding becomes a halo exchange
    (zeros at the poles), the circular padding of W stays."""

    def __init__(self, periodic_conv, shard_dim: int = -2, dom=None):
        super().__init__()
        self.conv, self.padding = periodic_conv.conv, int(periodic_conv.padding)
        self.halo = HaloExchange(self.padding, shard_dim, dom)

    def forward(self, x):
        x = F.pad(x, (self.padding, self.padding, 0, 0), mode="circular")
        if not self.halo.dom.active:
            x = F.pad(x, (0, 0, self.padding, self.padding), mode="reflect")
            return self.conv(x)
        return self.conv(self.halo(x))

    @property
    def weight(self):
        return self.conv.weight

    @property
    def bias(self):
        return self.conv.bias


class DomainParallelInterpolate(nn.Module):
    """Interpolation to ``size`` (the *local* target extent): one halo row on each side so that rows next to the cut
    interpolate against their true neighbours, the target extent scaled accordingly, the surplus rows trimmed."""

    def __init__(self, size, mode: str = "bilinear", shard_dim: int = -2, dom=None):
        super().__init__()
        self.size, self.mode = size, mode
        self.halo = HaloExchange(1, shard_dim, dom)

    def forward(self, x):
        kw = {} if self.mode in ("nearest", "area", "nearest-exact") else {"align_corners": False}
        if not self.halo.dom.active:
            return F.interpolate(x, size=self.size, mode=self.mode, **kw)
        h_target, w_target = (self.size if isinstance(self.size, (tuple, list)) else (self.size, self.size))
        padded = self.halo(x)
        h_scaled = int(h_target * padded.shape[-2] / x.shape[-2])
        out = F.interpolate(padded, size=(h_scaled, w_target), mode=self.mode, **kw)
        cut = (h_scaled - h_target) // 2
        return out[:, :, cut:cut + h_target, :] if cut > 0 else out


# ------------------------------------------------------------------------------------------------ conversion
def _crosses_cut(conv, axis) -> bool:
    return _component(conv.kernel_size, axis) > 1


def _overlaps(conv, axis) -> bool:
    return _component(conv.kernel_size, axis) > _component(conv.stride, axis)


def convert_to_domain_parallel(model: nn.Module, dom, shard_dim: int = -2,
                               custom_converters: Optional[Dict[type, Callable[[nn.Module], nn.Module]]] = None) -> nn.Module:
    """Replace, in place, every layer of ``model`` whose result depends on rows across the cut: ``nn.Conv2d`` /
    ``nn.Conv3d`` with a kernel wider than one row, ``nn.ConvTranspose2d`` / ``3d`` whose kernel exceeds the stride, and
    every ``nn.GroupNorm``. 1 x 1 convolutions, channel-wise norms, activations and the like are left alone.
    ``custom_converters``: ``{module type: callable(module) -> replacement}``, tried first; the children of a module
    replaced this way are not visited (for wrappers such as a periodic convolution that own an inner ``nn.Conv2d``).
    Returns the model; ``model.domain_parallel_counts`` holds how many layers of each kind were replaced."""
    d = _dom(dom)
    custom = custom_converters or {}
    counts = {"conv2d": 0, "conv3d": 0, "conv_transpose2d": 0, "conv_transpose3d": 0, "group_norm": 0, "custom": 0}
    axis2 = (shard_dim % 4) - 2
    shard_dim_5d = 3

    def replacement(m):
        for kind, make in custom.items():
            if isinstance(m, kind):
                counts["custom"] += 1
                return make(m)
        if isinstance(m, nn.Conv2d) and _crosses_cut(m, axis2):
            counts["conv2d"] += 1
            return DomainParallelConv2d(m, shard_dim, d)
        if isinstance(m, nn.Conv3d) and _crosses_cut(m, shard_dim_5d - 2):
            counts["conv3d"] += 1
            return DomainParallelConv3d(m, shard_dim_5d, d)
        if isinstance(m, nn.ConvTranspose2d) and _overlaps(m, axis2):
            counts["conv_transpose2d"] += 1
            return DomainParallelConvTranspose2d(m, shard_dim, d)
        if isinstance(m, nn.ConvTranspose3d) and _overlaps(m, shard_dim_5d - 2):
            counts["conv_transpose3d"] += 1
            return DomainParallelConvTranspose3d(m, shard_dim_5d, d)
        if isinstance(m, nn.GroupNorm):
            counts["group_norm"] += 1
            return DomainParallelGroupNorm(m, d)
        return None

    def walk(parent):
        for name, child in list(parent.named_children()):
            new = replacement(child)
            if new is not None:
                setattr(parent, name, new)
            else:
                walk(child)

    walk(model)
    model.domain_parallel_counts = counts
    return model


def validate_sharding_constraints(model, local_h: int, window_sizes=None) -> List[str]:
    """Warnings for a local extent that the model's windows do not divide, level by level (each level halves H)."""
    notes = []
    if window_sizes is not None:
        h = local_h
        for level, ws in enumerate(window_sizes):
            ws_h = ws[0] if isinstance(ws, (tuple, list)) else ws
            if h % ws_h != 0:
                notes.append(f"Level {level}: local H={h} not divisible by window_size={ws_h}. Attention will fail. "
                             "Consider adjusting the number of domain-parallel ranks or the padding.")
            h //= 2
    return notes
