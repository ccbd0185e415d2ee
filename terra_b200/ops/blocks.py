"""Fused transformer-block operators.

On CUDA each Swin half-block is one autograd node built from the sm_100a kernels:

  attention half:  LN -> [q|k|v] GEMM (one [3C, C] operand) -> window attention -> proj GEMM (+bias +shortcut)
  MLP half:        LN -> fc1 GEMM (+bias, GELU, pre-activation kept) -> fc2 GEMM (+bias +shortcut)

Backward runs the transposed products on the same tcgen05 kernel (weights read MN-major for input gradients,
both operands MN-major with split-K fp32 atomics for weight gradients, accumulated straight into the flat
gradient arena), fuses GELU' into the fc2 input-gradient epilogue and the shortcut gradient into the LayerNorm
backward. On CPU the same math is plain PyTorch (autograd does the rest); that path is the oracle of the tests.

What these nodes compute is the reference's block halves: models/transformer.py:71-160 (``SequentialSwinTransformer``),
:963-1036 (window-parallel forward), models/attention.py:874-910 (window attention), models/mlp.py:138-175, 375-412 (MLP).
"""
from __future__ import annotations

import os

from typing import Optional

import torch
import torch.nn.functional as TF

from .. import _ext
from .attention import (MAX_KERNEL_WINDOW_TOKENS, WindowGeometry, launch_window_attn_bwd, launch_window_attn_fwd,
                        window_attention)
from .gemm import gemm, status_word
from .packed import fp32_values
from ..utils.nvtx import nvtx_range

LN_EPS = 1e-5


# Bias gradients come out of the weight-gradient GEMM itself (3 ms of an 88 ms step against the separate column-sum
# kernel, measured back to back on one GPU); TERRA_FUSED_BIAS_GRAD=0 restores the separate kernel.
FUSE_BIAS_GRAD = os.environ.get("TERRA_FUSED_BIAS_GRAD", "1") == "1"


def _split_k_for(m_tiles_n_tiles: int, k_blocks: int, sms: int = 148) -> int:
    """Enough K splits to fill the GPU once, never more than the number of 64-wide k-blocks."""
    want = max(1, sms // max(1, m_tiles_n_tiles))
    return max(1, min(want, k_blocks))


def wgrad_accumulate(dy: torch.Tensor, x: torch.Tensor, grad_w: torch.Tensor, grad_b: torch.Tensor = None) -> None:
    """grad_w[N, K] (fp32) += dy[M, N]^T @ x[M, K]; with ``grad_b``: grad_b[N] (fp32) += column sums of dy, from the
    same kernel (a 16-column MMA of the dy tiles against ones), which saves the separate pass over dy."""
    N, K = grad_w.shape
    if grad_b is not None and not FUSE_BIAS_GRAD:
        bias_grad_accumulate(dy, grad_b)
        grad_b = None
    wide = K % 256 == 0 and K >= 1024 and (grad_b is None or K % 192 != 0)     # the sums need tile widths <= 192
    bn = 256 if wide else (192 if K % 192 == 0 else 128)
    tiles = ((N + 127) // 128) * ((K + bn - 1) // bn)
    split = _split_k_for(tiles, (dy.shape[0] + 63) // 64)
    if grad_b is not None and bn == 256:
        bias_grad_accumulate(dy, grad_b)
        grad_b = None
    gemm(dy, x, a_mn=True, b_mn=True, out=grad_w, accumulate=True, split_k=split, bn=bn, colsum=grad_b)


def bias_grad_accumulate(dy: torch.Tensor, grad_b: torch.Tensor) -> None:
    _ext.load().colsum(dy, grad_b)


@nvtx_range("terra.layernorm")
def layernorm_cuda(x, w16, b16):
    ext = _ext.load()
    y = torch.empty_like(x)
    mean = torch.empty(x.shape[0], dtype=torch.float32, device=x.device)
    rstd = torch.empty_like(mean)
    ext.layernorm_fwd(x, w16, b16, y, mean, rstd, LN_EPS)
    return y, mean, rstd


def layernorm_bwd_cuda(dy, x, w16, mean, rstd, grad_w, grad_b, dres=None):
    ext = _ext.load()
    dx = torch.empty_like(x)
    ext.layernorm_bwd(dy, x, w16, mean, rstd, dx, grad_w, grad_b, dres)
    return dx


class ParamPack:
    """bf16 value + fp32 gradient-accumulator views of the parameters one fused block needs."""

    def __init__(self, **kw):
        self.__dict__.update(kw)


def _views(p: torch.nn.Parameter):
    if getattr(p, "bf16", None) is None:
        raise RuntimeError("CUDA path needs flattened parameters: call terra_b200.utils.flat_params.ParamArena(model)")
    return p.bf16, p.grad


class _AttnHalfFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, anchor, pk: ParamPack, geo: WindowGeometry, num_heads, shifted, use_mask, scale, comm):
        ext = _ext.load()
        C = x.shape[1]
        xn, mean, rstd = layernorm_cuda(x, pk.ln_w, pk.ln_b)
        if comm is not None:
            qkv = comm.alloc_qkv(x.shape[0], 3 * C)
            gemm(xn, pk.qkv_w, bias=pk.qkv_b, out=qkv)
            o, qkv_ptrs, out_ptrs = comm.attn_forward_buffers(qkv, C, shifted)
        else:
            qkv = gemm(xn, pk.qkv_w, bias=pk.qkv_b)
            o = torch.empty(x.shape[0], C, dtype=torch.bfloat16, device=x.device)
            qkv_ptrs, out_ptrs = [qkv.data_ptr()], [o.data_ptr()]
        sh, sw = geo.shift(shifted)
        launch_window_attn_fwd(ext, qkv_ptrs, out_ptrs, pk.bias_table, geo, C, num_heads, sh, sw, use_mask and shifted,
                               scale, x.device)
        if comm is not None:
            o, qkv = comm.attn_forward_done(o, qkv, shifted)
        y = gemm(o, pk.proj_w, bias=pk.proj_b, residual=x)
        ctx.save_for_backward(x, mean, rstd, xn, qkv, o)
        ctx.pk, ctx.geo, ctx.args, ctx.comm = pk, geo, (num_heads, shifted, use_mask, scale), comm
        return y

    @staticmethod
    def backward(ctx, dy):
        ext = _ext.load()
        x, mean, rstd, xn, qkv, o = ctx.saved_tensors
        pk, geo, comm = ctx.pk, ctx.geo, ctx.comm
        num_heads, shifted, use_mask, scale = ctx.args
        C = x.shape[1]
        dy = dy.contiguous()
        wgrad_accumulate(dy, o, pk.proj_wg, pk.proj_bg)
        if comm is not None:
            do = comm.alloc_dout(x.shape[0], C)
            gemm(dy, pk.proj_w, b_mn=True, out=do)
            dqkv, qkv_ptrs, dout_ptrs, dqkv_ptrs = comm.attn_backward_buffers(qkv, do, shifted)
        else:
            do = gemm(dy, pk.proj_w, b_mn=True)
            dqkv = torch.empty_like(qkv)
            qkv_ptrs, dout_ptrs, dqkv_ptrs = [qkv.data_ptr()], [do.data_ptr()], [dqkv.data_ptr()]
        sh, sw = geo.shift(shifted)
        launch_window_attn_bwd(ext, qkv_ptrs, dout_ptrs, dqkv_ptrs, pk.bias_table, pk.bias_table_g, geo, C, num_heads, sh, sw,
                               use_mask and shifted, scale, x.device)
        if comm is not None:
            dqkv = comm.attn_backward_done(dqkv, shifted)
        wgrad_accumulate(dqkv, xn, pk.qkv_wg, pk.qkv_bg)
        dxn = gemm(dqkv, pk.qkv_w, b_mn=True)
        dx = layernorm_bwd_cuda(dxn, x, pk.ln_w, mean, rstd, pk.ln_wg, pk.ln_bg, dres=dy)
        return dx, None, None, None, None, None, None, None, None


class _MlpHalfFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, anchor, pk: ParamPack):
        xn, mean, rstd = layernorm_cuda(x, pk.ln_w, pk.ln_b)
        act, pre = gemm(xn, pk.fc1_w, bias=pk.fc1_b, gelu=True, save_pre=True, bn=256 if pk.fc1_w.shape[0] % 256 == 0 else 0)
        y = gemm(act, pk.fc2_w, bias=pk.fc2_b, residual=x)
        ctx.save_for_backward(x, mean, rstd, xn, pre, act)
        ctx.pk = pk
        return y

    @staticmethod
    def backward(ctx, dy):
        x, mean, rstd, xn, pre, act = ctx.saved_tensors
        pk = ctx.pk
        dy = dy.contiguous()
        wgrad_accumulate(dy, act, pk.fc2_wg, pk.fc2_bg)
        dpre = gemm(dy, pk.fc2_w, b_mn=True, dgelu_aux=pre, bn=256 if pk.fc2_w.shape[1] % 256 == 0 else 0)
        wgrad_accumulate(dpre, xn, pk.fc1_wg, pk.fc1_bg)
        dxn = gemm(dpre, pk.fc1_w, b_mn=True)
        dx = layernorm_bwd_cuda(dxn, x, pk.ln_w, mean, rstd, pk.ln_wg, pk.ln_bg, dres=dy)
        return dx, None, None


class _LinearFn(torch.autograd.Function):
    """y = x @ W^T + b (+ residual). ``anchor`` is any parameter: it makes autograd call backward even when the
    activation input carries no gradient (first layer)."""

    @staticmethod
    def forward(ctx, x, anchor, w16, b16, wg, bg, residual, need_dx):
        y = gemm(x, w16, bias=b16, residual=residual)
        ctx.save_for_backward(x)
        ctx.p = (w16, wg, bg, residual is not None, need_dx)
        return y

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        w16, wg, bg, has_res, need_dx = ctx.p
        dy = dy.contiguous()
        wgrad_accumulate(dy, x, wg, bg)
        dx = gemm(dy, w16, b_mn=True) if need_dx else None
        return dx, None, None, None, None, None, (dy if has_res else None), None


class LayerNormFn(torch.autograd.Function):
    """Standalone LayerNorm on the CUDA kernels (where the norm is not fused into a block half: in front of a
    collective, or for windows too large for the fused attention half). ``weight`` / ``bias`` are arena parameters;
    their gradients are accumulated in place."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        y, mean, rstd = layernorm_cuda(x, weight.bf16, bias.bf16)
        ctx.save_for_backward(x, mean, rstd)
        ctx.p = (weight, bias)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, mean, rstd = ctx.saved_tensors
        weight, bias = ctx.p
        dx = layernorm_bwd_cuda(dy.contiguous(), x, weight.bf16, mean, rstd, weight.grad, bias.grad)
        return dx, None, None


# ------------------------------------------------------------------------------------------------ public entry points
@nvtx_range("terra.attention_half")
def attention_half(x, mod, geo: WindowGeometry, shifted: bool, comm=None):
    """x + proj(window_attention(qkv(norm1(x)))) for a ``SwinAttentionHalf`` module ``mod``."""
    if x.is_cuda and geo.N > MAX_KERNEL_WINDOW_TOKENS:
        # large windows: the fused half needs the shared-memory kernel; compose the half from its parts instead
        a = mod.attn
        xn = LayerNormFn.apply(x.contiguous(), mod.norm1.weight, mod.norm1.bias)
        qkv = torch.cat([linear(xn, a.q_linear), linear(xn, a.k_linear), linear(xn, a.v_linear)], dim=-1)
        o = window_attention(qkv, geo, a.num_heads, shifted, a.bias_table(), mod.use_attn_mask, a.scale, comm)
        return linear(o.to(x.dtype).contiguous(), a.proj, residual=x)
    if x.is_cuda:
        fused = getattr(mod.attn, "fused", None)
        if fused is None:
            raise RuntimeError("CUDA path needs flattened parameters (ParamArena)")
        has_bias = mod.attn.use_relative_position_bias
        pk = ParamPack(
            ln_w=mod.norm1.weight.bf16, ln_b=mod.norm1.bias.bf16, ln_wg=mod.norm1.weight.grad, ln_bg=mod.norm1.bias.grad,
            qkv_w=fused["qkv_weight"].bf16, qkv_b=fused["qkv_bias"].bf16, qkv_wg=fused["qkv_weight"].grad,
            qkv_bg=fused["qkv_bias"].grad,
            proj_w=mod.attn.proj.weight.bf16, proj_b=mod.attn.proj.bias.bf16, proj_wg=mod.attn.proj.weight.grad,
            proj_bg=mod.attn.proj.bias.grad,
            bias_table=fp32_values(mod.attn.relative_position_bias_table) if has_bias else None,
            bias_table_g=mod.attn.relative_position_bias_table.grad if has_bias else None)
        return _AttnHalfFn.apply(x, mod.norm1.weight, pk, geo, mod.attn.num_heads, shifted, mod.use_attn_mask,
                                 mod.attn.scale, comm)
    a = mod.attn
    xn = TF.layer_norm(x, (x.shape[-1],), mod.norm1.weight, mod.norm1.bias, LN_EPS)
    qkv = torch.cat([a.q_linear(xn), a.k_linear(xn), a.v_linear(xn)], dim=-1)
    o = window_attention(qkv, geo, a.num_heads, shifted, a.bias_table(), mod.use_attn_mask, a.scale, comm)
    return x + a.proj(o)


@nvtx_range("terra.mlp_half")
def mlp_half(x, mod):
    """x + fc2(gelu(fc1(norm2(x))))."""
    if x.is_cuda:
        pk = ParamPack(
            ln_w=mod.norm2.weight.bf16, ln_b=mod.norm2.bias.bf16, ln_wg=mod.norm2.weight.grad, ln_bg=mod.norm2.bias.grad,
            fc1_w=mod.fc1.weight.bf16, fc1_b=mod.fc1.bias.bf16, fc1_wg=mod.fc1.weight.grad, fc1_bg=mod.fc1.bias.grad,
            fc2_w=mod.fc2.weight.bf16, fc2_b=mod.fc2.bias.bf16, fc2_wg=mod.fc2.weight.grad, fc2_bg=mod.fc2.bias.grad)
        return _MlpHalfFn.apply(x, mod.norm2.weight, pk)
    xn = TF.layer_norm(x, (x.shape[-1],), mod.norm2.weight, mod.norm2.bias, LN_EPS)
    return x + mod.fc2(TF.gelu(mod.fc1(xn)))


def linear(x, lin: torch.nn.Linear, residual=None, need_dx=True):
    """2-D ``x``; on CUDA runs the tcgen05 GEMM with the bias (and residual) fused."""
    if x.is_cuda:
        w16, wg = _views(lin.weight)
        b16, bg = _views(lin.bias) if lin.bias is not None else (None, None)
        return _LinearFn.apply(x, lin.weight, w16, b16, wg, bg, residual, need_dx)
    y = TF.linear(x, lin.weight, lin.bias)
    return y if residual is None else y + residual
