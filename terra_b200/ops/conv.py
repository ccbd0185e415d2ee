"""FuXi-style sampling-block operators on NHWC activations.

CUDA: 3x3 convolutions (stride 1 / 2, padding 1) are implicit GEMMs on the tcgen05 kernel - the A operand is
gathered by 5-D TMA boxes with zero fill outside the image, k-blocks enumerate (tap, channel chunk); the input
gradient of the stride-1 convolution is the same kernel with flipped, transposed weights; weight gradients
contract over pixels with one tile group per tap. The 2x2/stride-2 transposed convolution is a GEMM whose
epilogue stores pixel-shuffled. GroupNorm+SiLU is a statistics pass plus one fused apply pass (optionally adding
the block's shortcut), its backward a reduce pass plus an apply pass.

With row-stripe domain parallelism (``dom`` given) halo rows come from the neighbours and GroupNorm statistics
are summed over the stripe group, so that the result equals the single-rank one.
CPU: plain PyTorch on the same NHWC tensors (oracle for the tests, gloo ranks for the multi-rank logic).

Reference: models/utils.py:101-180 (``CreditDownBlock`` / ``CreditUpBlock``), credit/domain_parallel/layers.py:18-84,
87-208, 429-483 and halo_exchange.py:18-157 for the row-stripe forms.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as TF

from .. import _ext
from . import _flags as F
from .gemm import gemm, status_word
from .packed import PACK_EPOCH, _packed, fp32_values, invalidate_packed_weights  # noqa: F401  (re-exported)
from .blocks import FUSE_BIAS_GRAD, wgrad_accumulate, bias_grad_accumulate
from ..utils.nvtx import nvtx_range

GN_EPS = 1e-5


# ------------------------------------------------------------------------------------------------ weight packing
def pack_conv3x3_weight(w: torch.Tensor) -> torch.Tensor:
    """(Cout, Cin, 3, 3) -> bf16 [Cout, 9 * Cin_pad], tap-major, Cin padded to a multiple of 64 with zeros."""
    cout, cin = w.shape[:2]
    cpad = (cin + 63) // 64 * 64
    wp = torch.zeros(cout, 9, cpad, device=w.device, dtype=torch.bfloat16)
    wp[:, :, :cin] = w.permute(0, 2, 3, 1).reshape(cout, 9, cin)
    return wp.view(cout, 9 * cpad)


def pack_conv3x3_weight_dgrad(w: torch.Tensor) -> torch.Tensor:
    """Weights of the stride-1 input-gradient convolution: taps flipped, channels swapped."""
    return pack_conv3x3_weight(w.flip(2, 3).transpose(0, 1))




_SCRATCH = {}


def _zero_scratch(device, shape, tag):
    """Persistent fp32 staging that is handed out zeroed and comes back zeroed (its consumer clears it behind the
    read), so that no fill kernel runs per use."""
    key = (torch.device(device).index, tuple(shape), tag)
    buf = _SCRATCH.get(key)
    if buf is None:
        buf = torch.zeros(*shape, device=device, dtype=torch.float32)
        _SCRATCH[key] = buf
    return buf


def _arena_grad(p):
    """The parameter's fp32 gradient view in the flat arena (accumulated into in place), or None."""
    g = getattr(p, "grad", None)
    if g is not None and g.is_cuda and g.dtype == torch.float32 and g.is_contiguous() and getattr(p, "bf16", None) is not None:
        return g
    return None


class _Conv3x3Fn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, stride, dom):
        ext = _ext.load()
        B, H, W, Cin = x.shape
        Cout = weight.shape[0]
        Ho, Wo = (H, W) if stride == 1 else ((H + 1) // 2, W // 2)
        y = torch.empty(B, Ho, Wo, Cout, device=x.device, dtype=torch.bfloat16)
        w16 = weight.bf16 if getattr(weight, "bf16", None) is not None else weight.detach().to(torch.bfloat16)
        b16 = bias.bf16 if getattr(bias, "bf16", None) is not None else bias.detach().to(torch.bfloat16)
        wp = _packed(weight, w16, "fwd", pack_conv3x3_weight)
        multi = dom is not None and dom.world > 1
        lo, hi = dom.exchange_rows(x) if multi else (None, None)
        ext.conv3x3_fwd(x, wp, y, stride, F.EPI_BIAS, b16, None, status_word(x.device), lo, hi)
        ctx.save_for_backward(x)
        ctx.p = (weight, bias, w16, stride, dom, lo, hi)
        return y

    @staticmethod
    def backward(ctx, dy):
        ext = _ext.load()
        (x,) = ctx.saved_tensors
        weight, bias, w16, stride, dom, lo, hi = ctx.p
        multi = dom is not None and dom.world > 1
        dy = dy.contiguous()
        B, H, W, Cin = x.shape
        Cout = weight.shape[0]
        # ---- weight / bias gradients (fp32); the halo rows received in forward serve the boundary taps
        gw, gb = _arena_grad(weight), _arena_grad(bias)
        if gw is not None:
            # tap-major staging [9, Cout, Cin] (persistent, self-cleaning) folded into the arena's (Cout, Cin, 3, 3) view
            dw9 = _zero_scratch(x.device, (9, Cout, Cin), "conv3x3")
            # the bias gradient (column sums of dy) comes out of the same kernel
            ext.conv3x3_wgrad(x, dy, dw9, stride, _wgrad_split(B, H, W, stride, Cout, Cin), status_word(x.device), lo, hi,
                              bias_grad=gb if FUSE_BIAS_GRAD else None)
            ext.strided_add(dw9, gw, 1, Cin * 9, 9, True)
            dw = None
        else:
            dw9 = torch.zeros(9, Cout, Cin, device=x.device, dtype=torch.float32)
            ext.conv3x3_wgrad(x, dy, dw9, stride, _wgrad_split(B, H, W, stride, Cout, Cin), status_word(x.device), lo, hi)
            dw = dw9.view(3, 3, Cout, Cin).permute(2, 3, 0, 1)
        if gb is not None:
            if gw is None or not FUSE_BIAS_GRAD:
                ext.colsum(dy.view(-1, Cout), gb)
            db = None
        else:
            db = torch.zeros(Cout, device=x.device, dtype=torch.float32)
            ext.colsum(dy.view(-1, Cout), db)
        # ---- input gradient
        dx = None
        if ctx.needs_input_grad[0]:
            if stride == 1:
                dx = torch.empty_like(x)
                wf = _packed(weight, w16, "dgrad", pack_conv3x3_weight_dgrad)
                glo, ghi = dom.exchange_rows(dy) if multi else (None, None)
                ext.conv3x3_fwd(dy, wf, dx, 1, 0, None, None, status_word(x.device), glo, ghi)
            else:
                dx = _conv3x3_s2_dgrad(dy, w16, H, W, dom, weight)
        return dx, dw, db, None, None


def balanced_split(tiles: int, kblocks: int, sms: int = 148, limit: int = 64) -> int:
    """Split-K factor for a persistent kernel of ``sms`` CTAs: the one whose ``tiles * split`` work items fill whole
    rounds of CTAs best (time ~ ceil(tiles * split / sms) / split), the smaller factor on near ties (every split adds
    one pass of fp32 atomics over the output)."""
    best, best_cost = 1, float("inf")
    for s in range(1, max(1, min(kblocks, limit)) + 1):
        cost = -(-tiles * s // sms) / s + 0.002 * s
        if cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


def _wgrad_split(B, H, W, stride, Cout, Cin):
    Ho, Wo = (H, W) if stride == 1 else ((H + 1) // 2, W // 2)
    kblocks = B * Ho * ((Wo + 63) // 64)
    bn = 192 if Cin % 192 == 0 else 128            # the tile width conv3x3_wgrad picks
    tiles = 9 * ((Cout + 127) // 128) * ((Cin + bn - 1) // bn)
    return balanced_split(tiles, kblocks)


def _conv3x3_s2_dgrad(dy, w16, H, W, dom, weight=None):
    """Input gradient of the stride-2 convolution: dcol = dy @ W (tap-major columns) on the tcgen05 GEMM,
    then one gather kernel over the (at most four) taps that reach each input pixel."""
    B, Ho, Wo, Cout = dy.shape
    Cin = w16.shape[1]
    build = lambda w: w.permute(0, 2, 3, 1).reshape(Cout, 9 * Cin).contiguous()          # [Cout, (tap, ci)]
    wk = _packed(weight, w16, "s2dgrad", build) if weight is not None else build(w16)
    dcol = gemm(dy.view(-1, Cout), wk, b_mn=True).view(B, Ho, Wo, 9, Cin)     # dcol[p, tap, ci]
    ext = _ext.load()
    if dom is not None and dom.world > 1:
        # the rows above / below the stripe (padded rows 0 and H + 1) receive gradient too: it goes back to the
        # neighbours, so the padded rows are produced (fp32, as the halo fold accumulates)
        dxp = torch.zeros(B, H + 2, W + 2, Cin, device=dy.device, dtype=torch.float32)
        inner = torch.empty(B, H + 2, W, Cin, device=dy.device, dtype=torch.float32)
        ext.conv_s2_col2im(dcol.contiguous(), inner, W, 0)
        dxp[:, :, 1:W + 1] = inner
        return dom.fold_halo_grad(dxp, H, W).to(torch.bfloat16).contiguous()
    out = torch.empty(B, H, W, Cin, device=dy.device, dtype=torch.bfloat16)
    ext.conv_s2_col2im(dcol.contiguous(), out, W, 1)
    return out


@nvtx_range("terra.conv3x3")
def conv3x3(x, conv: torch.nn.Conv2d, stride: int = 1, dom=None):
    """x NHWC -> NHWC. ``conv`` holds a (Cout, Cin, 3, 3) weight and a bias."""
    if x.is_cuda:
        return _Conv3x3Fn.apply(x, conv.weight, conv.bias, stride, dom)
    xin = x.permute(0, 3, 1, 2)
    if dom is not None and dom.world > 1:
        xin = dom.halo_exchange_cpu(xin, 1)
        y = TF.conv2d(xin, conv.weight, conv.bias, stride=stride, padding=(0, 1))
        if stride == 2 and y.shape[2] > (x.shape[1] + 1) // 2:
            y = y[:, :, :(x.shape[1] + 1) // 2]
    else:
        y = TF.conv2d(xin, conv.weight, conv.bias, stride=stride, padding=1)
    return y.permute(0, 2, 3, 1)


# ------------------------------------------------------------------------------------------------ transposed conv 2x2 / s2
class _ConvT2x2Fn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        ext = _ext.load()
        B, H, W, Cin = x.shape
        Cout = weight.shape[1]
        w16 = weight.bf16 if getattr(weight, "bf16", None) is not None else weight.detach().to(torch.bfloat16)
        b16 = bias.bf16 if getattr(bias, "bf16", None) is not None else bias.detach().to(torch.bfloat16)
        wt = _packed(weight, w16, "convT", lambda w: w.permute(2, 3, 1, 0).reshape(4 * Cout, Cin).contiguous())   # [(dy, dx, co), ci]
        b4 = _packed(bias, b16, "convT_bias", lambda b: b.repeat(4))
        y = torch.empty(B, 2 * H, 2 * W, Cout, device=x.device, dtype=torch.bfloat16)
        x2 = x.view(-1, Cin)
        bn = 128 if Cout % 128 == 0 else (64 if Cout % 64 == 0 else 0)
        if bn:
            # every BN-wide column tile lies inside one (dy, dx) phase: the epilogue stores it pixel-shuffled
            flags = F.EPI_BIAS | F.EPI_ROW_SHUFFLE
            ext.gemm(x2, False, wt, False, y.view(-1, Cout), flags, b4, None, None, None, 1.0, 1, bn,
                     status_word(x.device), Cout, W, H, 0, [], 0, [], 0, 0, 0, 1, 1)
        else:
            flat = gemm(x2, wt, bias=b4)
            y.copy_(flat.view(B, H, W, 2, 2, Cout).permute(0, 1, 3, 2, 4, 5).reshape(B, 2 * H, 2 * W, Cout))
        ctx.save_for_backward(x)
        ctx.p = (wt, Cout, weight, bias)
        return y

    @staticmethod
    def backward(ctx, dy):
        ext = _ext.load()
        (x,) = ctx.saved_tensors
        wt, Cout, weight, bias = ctx.p
        B, H, W, Cin = x.shape
        # un-shuffle dy to [pixels, (dy, dx, co)] once; both products read it
        dyu = dy.view(B, H, 2, W, 2, Cout).permute(0, 1, 3, 2, 4, 5).reshape(B * H * W, 4 * Cout)
        gw, gb = _arena_grad(weight), _arena_grad(bias)
        if gw is not None:
            dwt = _zero_scratch(x.device, (4 * Cout, Cin), "convT")
            wgrad_accumulate(dyu, x.view(-1, Cin), dwt)
            # [(tap), co, ci] staging -> (Cin, Cout, 2, 2) arena view
            ext.strided_add(dwt.view(4, Cout, Cin), gw, 1, 4, Cout * 4, True)
            dw = None
        else:
            dwt = torch.zeros(4 * Cout, Cin, device=x.device, dtype=torch.float32)
            wgrad_accumulate(dyu, x.view(-1, Cin), dwt)
            dw = dwt.view(2, 2, Cout, Cin).permute(3, 2, 0, 1)
        if gb is not None:
            ext.colsum(dy.reshape(-1, Cout), gb)
            db = None
        else:
            db = torch.zeros(Cout, device=x.device, dtype=torch.float32)
            ext.colsum(dy.reshape(-1, Cout), db)
        dx = gemm(dyu, wt, b_mn=True).view(B, H, W, Cin) if ctx.needs_input_grad[0] else None
        return dx, dw, db


def conv_transpose2x2(x, convt: torch.nn.ConvTranspose2d):
    if x.is_cuda:
        return _ConvT2x2Fn.apply(x, convt.weight, convt.bias)
    return TF.conv_transpose2d(x.permute(0, 3, 1, 2), convt.weight, convt.bias, stride=2).permute(0, 2, 3, 1)


# ------------------------------------------------------------------------------------------------ GroupNorm + SiLU
class _GroupNormSiluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, residual, groups, dom):
        ext = _ext.load()
        B, H, W, C = x.shape
        x3 = x.view(B, H * W, C)
        multi = dom is not None and dom.world > 1
        count = float(H * W * (C // groups)) * (dom.world if multi else 1)
        stats = torch.empty(B, groups, 2, device=x.device, dtype=torch.float32)
        if multi:
            sums = torch.zeros(B, groups, 2, device=x.device, dtype=torch.float32)
            ext.groupnorm_stats(x3, sums, groups)
            sums = dom.all_reduce_small(sums)
            ext.groupnorm_finalize(sums, stats, 1.0 / count, GN_EPS, False)
        else:
            sums = _zero_scratch(x.device, (B, groups, 2), "gn_sums")          # cleared again by the finalize kernel
            ext.groupnorm_stats(x3, sums, groups)
            ext.groupnorm_finalize(sums, stats, 1.0 / count, GN_EPS, True)
        g16 = gamma.bf16 if getattr(gamma, "bf16", None) is not None else gamma.detach().to(torch.bfloat16)
        b16 = beta.bf16 if getattr(beta, "bf16", None) is not None else beta.detach().to(torch.bfloat16)
        y = torch.empty_like(x)
        ext.groupnorm_silu_apply(x3, stats, g16, b16, None if residual is None else residual.view(B, H * W, C),
                                 y.view(B, H * W, C), groups)
        ctx.save_for_backward(x, stats, g16, b16)
        ctx.p = (groups, dom, count, residual is not None, gamma, beta)
        return y

    @staticmethod
    def backward(ctx, dy):
        ext = _ext.load()
        x, stats, g16, b16 = ctx.saved_tensors
        groups, dom, count, has_res, gamma, beta = ctx.p
        B, H, W, C = x.shape
        dy = dy.contiguous()
        x3, dy3 = x.view(B, H * W, C), dy.view(B, H * W, C)
        red = torch.zeros(B, C, 2, device=x.device, dtype=torch.float32)
        gg, gbt = _arena_grad(gamma), _arena_grad(beta)
        if gg is not None and gbt is not None:
            # the affine parameters' gradients are accumulated by the reduce kernel itself
            ext.groupnorm_silu_bwd_reduce(dy3, x3, stats, g16, b16, red, groups, gg, gbt)
            dgamma = dbeta = None
        else:
            ext.groupnorm_silu_bwd_reduce(dy3, x3, stats, g16, b16, red, groups)
            dgamma, dbeta = red[..., 1].sum(0), red[..., 0].sum(0)
        if dom is not None and dom.world > 1:
            red = dom.all_reduce_small(red)
        dx = torch.empty_like(x)
        ext.groupnorm_silu_bwd_apply(dy3, x3, stats, red, g16, b16, dx.view(B, H * W, C), groups, 1.0 / count)
        return dx, dgamma, dbeta, (dy if has_res else None), None, None


def groupnorm_silu(x, gn: torch.nn.GroupNorm, residual=None, dom=None):
    """silu(group_norm(x)) [+ residual] on NHWC; statistics span the whole (global) image."""
    if x.is_cuda:
        return _GroupNormSiluFn.apply(x, gn.weight, gn.bias, residual, gn.num_groups, dom)
    xc = x.permute(0, 3, 1, 2)
    if dom is not None and dom.world > 1:
        y = dom.group_norm_cpu(xc, gn.num_groups, gn.weight, gn.bias, GN_EPS)
    else:
        y = TF.group_norm(xc, gn.num_groups, gn.weight, gn.bias, GN_EPS)
    y = TF.silu(y).permute(0, 2, 3, 1)
    return y if residual is None else y + residual
