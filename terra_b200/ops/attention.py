"""Swin window attention over the window-major activation layout.

``WindowGeometry`` describes one rank's slice of the global window grid. ``window_attention`` dispatches to
the sm_100a kernel (csrc/window_attn.cu) on CUDA tensors and to ``window_attention_reference`` (plain PyTorch,
also the numerical oracle of the tests) elsewhere.

Layout contract: activations are ``[B * nW_local * shardN, C]`` rows, windows in row-major order of the
rank's flat window range, tokens row-major inside the window, never shifted. For odd ("shifted") blocks the
roll by ``(-sh, -sw)``, the partition, the reverse and the roll back are index arithmetic
(reference semantics: models/transformer.py:976-1023, core/window_parallel.py:26-46).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from .. import _ext
from .packed import fp32_values
from ..utils.nvtx import nvtx_range


@dataclass
class WindowGeometry:
    B: int
    nWh: int
    nWw: int
    wh: int
    ww: int
    win_start: List[int] = field(default_factory=list)   # flat window range per window-group rank
    my_wg: int = 0
    sp: int = 1
    my_sp: int = 0
    tp: int = 1          # > 1: the q/k/v rows are the concatenation of tp chunks [B, ceil(nW/tp) windows] (TP all-gather)

    def __post_init__(self):
        if not self.win_start:
            self.win_start = [0, self.nWh * self.nWw]

    @property
    def N(self) -> int:
        return self.wh * self.ww

    @property
    def shardN(self) -> int:
        return (self.N + self.sp - 1) // self.sp

    @property
    def n_wg(self) -> int:
        return len(self.win_start) - 1

    @property
    def nW_local(self) -> int:
        return self.win_start[self.my_wg + 1] - self.win_start[self.my_wg]

    @property
    def rows_local(self) -> int:
        return self.B * self.nW_local * self.shardN

    def shift(self, shifted: bool):
        return (self.wh // 2, self.ww // 2) if shifted else (0, 0)


def relative_position_index(wh: int, ww: int) -> torch.Tensor:
    """[N, N] index into the ``(2wh-1)*(2ww-1)`` bias table (standard Swin)."""
    coords = torch.stack(torch.meshgrid(torch.arange(wh), torch.arange(ww), indexing="ij")).flatten(1)
    rel = coords[:, :, None] - coords[:, None, :]
    return (rel[0] + wh - 1) * (2 * ww - 1) + (rel[1] + ww - 1)


def region_ids(H: int, W: int, wh: int, ww: int, sh: int, sw: int) -> torch.Tensor:
    """[H, W] region id (0..8) of every position of the rolled frame (Swin SW-MSA mask regions)."""
    rh = torch.zeros(H, dtype=torch.long)
    rw = torch.zeros(W, dtype=torch.long)
    if sh > 0:
        rh[H - wh:H - sh] = 1
        rh[H - sh:] = 2
    if sw > 0:
        rw[W - ww:W - sw] = 1
        rw[W - sw:] = 2
    return rh[:, None] * 3 + rw[None, :]


def shifted_window_sources(geo: WindowGeometry, shifted: bool):
    """For every window of the shifted frame (all ``nWh*nWw`` of them) and token, the flat source window and
    source token in the unshifted frame, plus the token's mask region. Shapes ``[nW, N]``."""
    sh, sw = geo.shift(shifted)
    H, W = geo.nWh * geo.wh, geo.nWw * geo.ww
    hs = torch.arange(H)[:, None].expand(H, W)
    ws = torch.arange(W)[None, :].expand(H, W)
    gh = (hs + sh) % H
    gw = (ws + sw) % W
    src_win = (gh // geo.wh) * geo.nWw + (gw // geo.ww)
    src_tok = (gh % geo.wh) * geo.ww + (gw % geo.ww)
    reg = region_ids(H, W, geo.wh, geo.ww, sh, sw)

    def part(t):
        return t.view(geo.nWh, geo.wh, geo.nWw, geo.ww).permute(0, 2, 1, 3).reshape(geo.nWh * geo.nWw, geo.N)

    return part(src_win), part(src_tok), part(reg)


MAX_MMA_WINDOW_TOKENS = 128         # window_attn.cu (mma.sync forward / backward) keeps a whole window in shared memory
MAX_KERNEL_WINDOW_TOKENS = 128      # windows up to here run inside the fused attention half (LayerNorm .. proj in one node)


def attention_core_reference(q, k, v, scale, bias, mask):
    """q,k,v: [nWin, nH, Nq|N, hd] fp32; bias [nH, Nq, N] or None; mask [nWin, Nq, N] additive or None."""
    attn = (q * scale) @ k.transpose(-2, -1)
    if bias is not None:
        attn = attn + bias.unsqueeze(0)
    if mask is not None:
        attn = attn + mask.unsqueeze(1)
    return torch.softmax(attn, dim=-1) @ v


def attention_core_sdpa(q, k, v, scale, bias, mask):
    """Same contract as ``attention_core_reference`` on PyTorch's fused attention: no ``[N, N]`` score tensor is kept
    for autograd, and without bias and mask the flash kernel runs, so windows of thousands of tokens fit. Used for
    windows above the 128 tokens that ``window_attn.cu`` holds in shared memory."""
    add = None
    if bias is not None:
        add = bias.unsqueeze(0).to(q.dtype)
    if mask is not None:
        m = mask.unsqueeze(1).to(q.dtype)
        add = m if add is None else add + m
    return torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=add, scale=scale)


def window_attention_reference(qkv_all: torch.Tensor, geo: WindowGeometry, num_heads: int, shifted: bool,
                               bias_table: Optional[torch.Tensor], use_mask: bool, scale: float,
                               core=None) -> torch.Tensor:
    """Reference on the *global* window-major tensor ``[B, nW_total, N, 3C]`` -> ``[B, nW_total, N, C]``
    (single rank view; rows are gathered with explicit index tensors)."""
    B, nW, N = geo.B, geo.nWh * geo.nWw, geo.N
    C = qkv_all.shape[-1] // 3
    hd = C // num_heads
    src_win, src_tok, reg = shifted_window_sources(geo, shifted)
    flat_src = (src_win * N + src_tok).to(qkv_all.device)                       # [nW, N]
    x = qkv_all.reshape(B, nW * N, 3 * C)[:, flat_src.reshape(-1)].reshape(B, nW, N, 3, num_heads, hd)
    q, k, v = (x[:, :, :, i].permute(0, 1, 3, 2, 4).reshape(B * nW, num_heads, N, hd) for i in range(3))
    bias = None
    if bias_table is not None:
        idx = relative_position_index(geo.wh, geo.ww).to(bias_table.device)
        bias = bias_table[idx.reshape(-1)].reshape(N, N, num_heads).permute(2, 0, 1)
    mask = None
    if use_mask and shifted:
        reg = reg.to(qkv_all.device)
        mask = (reg[:, :, None] != reg[:, None, :]).to(q.dtype) * -100.0
        mask = mask.repeat(B, 1, 1)
    o = (core or attention_core_reference)(q, k, v, scale, bias, mask)          # [B*nW, nH, N, hd]
    o = o.permute(0, 2, 1, 3).reshape(B, nW * N, C)
    out = torch.empty_like(o)
    out[:, flat_src.reshape(-1)] = o
    return out.reshape(B, nW, N, C)


def attn_forward_impl(N: int) -> str:
    """Which forward kernel runs: ``tc`` (tcgen05 / TMEM, any window size) or ``mma`` (warp-level mma.sync, windows of
    at most 128 tokens, several CTAs per SM). Windows above 128 tokens always take ``tc``; below, ``mma`` is the default
    because it measures faster there (0.31 against 0.48 ms on the 2176-window stage with head dim 64): one softmax warp
    per scheduler leaves the tensor-core kernel latency bound on 64-token windows. ``TERRA_ATTN_FWD=tc`` selects it
    anyway."""
    import os

    if N > MAX_MMA_WINDOW_TOKENS:
        return "tc"
    return os.environ.get("TERRA_ATTN_FWD", "mma")


def attn_backward_impl(N: int, head_dim: int) -> str:
    """``tc``: the tcgen05 backward (two small windows per tile: N <= 64, head dim 16 / 32 / 64), ``mma``: the mma.sync
    one (N <= 128). Default ``mma`` (faster on small windows, see ``attn_forward_impl``); ``TERRA_ATTN_BWD=tc``."""
    import os

    want = os.environ.get("TERRA_ATTN_BWD", "mma")
    if want == "tc" and N <= 64 and head_dim in (16, 32, 64):
        return "tc"
    return "mma"


def launch_window_attn_fwd(ext, qkv_ptrs, out_ptrs, bias_f32, geo: "WindowGeometry", C, num_heads, sh, sw, use_mask, scale,
                           device, lse_ptrs=()):
    """One forward launch on the selected kernel (both take the same geometry)."""
    args = (list(geo.win_start), geo.my_wg, geo.sp, geo.my_sp, geo.shardN, geo.B, geo.nWh, geo.nWw, C, num_heads, geo.wh,
            geo.ww, sh, sw, bool(use_mask), float(scale), geo.tp)
    if attn_forward_impl(geo.N) == "tc":
        from .gemm import status_word

        ext.window_attn_tc_fwd(qkv_ptrs, out_ptrs, bias_f32, *args, status_word(device), list(lse_ptrs))
    else:
        ext.window_attn_fwd(qkv_ptrs, out_ptrs, bias_f32, *args)


def launch_window_attn_bwd(ext, qkv_ptrs, dout_ptrs, dqkv_ptrs, bias_f32, dbias, geo: "WindowGeometry", C, num_heads, sh, sw,
                           use_mask, scale, device, lse_ptrs=(), drow_ptrs=()):
    """One backward launch on the selected kernel. Windows above 128 tokens run the two-pass tensor-core backward,
    which needs the forward pass's log-sum-exp (``lse_ptrs``) and ``drow`` = rowsum(dO * O) per (row, head)."""
    args = (list(geo.win_start), geo.my_wg, geo.sp, geo.my_sp, geo.shardN, geo.B, geo.nWh, geo.nWw, C, num_heads, geo.wh,
            geo.ww, sh, sw, bool(use_mask), float(scale), geo.tp)
    hd = C // num_heads
    if geo.N > MAX_MMA_WINDOW_TOKENS:
        if hd not in (16, 32, 64):
            raise NotImplementedError(f"backward of windows above {MAX_MMA_WINDOW_TOKENS} tokens needs a head dim of 16, 32 "
                                      f"or 64 (got {hd})")
        from .gemm import status_word

        ext.window_attn_tc_bwd(qkv_ptrs, dout_ptrs, dqkv_ptrs, bias_f32, dbias, *args, status_word(device), list(lse_ptrs),
                               list(drow_ptrs))
    elif attn_backward_impl(geo.N, hd) == "tc":
        from .gemm import status_word

        ext.window_attn_tc_bwd(qkv_ptrs, dout_ptrs, dqkv_ptrs, bias_f32, dbias, *args, status_word(device), [], [])
    else:
        ext.window_attn_bwd(qkv_ptrs, dout_ptrs, dqkv_ptrs, bias_f32, dbias, *args)


def attention_forward(ext, qkv, geo: "WindowGeometry", C, num_heads, shifted, use_mask, scale, bias_f32, comm):
    """Forward on ``qkv`` (already in symmetric memory when ``comm`` is given). Returns ``(out, qkv, lse)``; ``lse``
    (fp32 ``[rows, heads]``, base 2) exists for windows above 128 tokens, whose backward needs it."""
    rows = qkv.shape[0]
    sh, sw = geo.shift(shifted)
    large = geo.N > MAX_MMA_WINDOW_TOKENS
    lse, lse_ptrs = None, ()
    if comm is None:
        out = torch.empty(rows, C, dtype=torch.bfloat16, device=qkv.device)
        qkv_ptrs, out_ptrs = [qkv.data_ptr()], [out.data_ptr()]
        if large:
            lse = torch.empty(rows, num_heads, dtype=torch.float32, device=qkv.device)
            lse_ptrs = [lse.data_ptr()]
    else:
        if large:
            lse = comm.alloc_f32(rows, num_heads)
            lse_ptrs = comm.arena.peer_ptrs(lse)
        out, qkv_ptrs, out_ptrs = comm.attn_forward_buffers(qkv, C, shifted)
    launch_window_attn_fwd(ext, qkv_ptrs, out_ptrs, bias_f32, geo, C, num_heads, sh, sw, use_mask and shifted, scale,
                           qkv.device, lse_ptrs)
    if comm is not None:
        out, qkv = comm.attn_forward_done(out, qkv, shifted)
    return out, qkv, lse


def attention_backward(ext, qkv, out, dout, lse, geo: "WindowGeometry", C, num_heads, shifted, use_mask, scale, bias_f32,
                       dbias, comm):
    """Gradient of ``qkv``. ``dout`` must already be in symmetric memory when ``comm`` is given."""
    sh, sw = geo.shift(shifted)
    large = geo.N > MAX_MMA_WINDOW_TOKENS
    drow, lse_ptrs, drow_ptrs = None, (), ()
    if large:
        drow = comm.alloc_f32(qkv.shape[0], num_heads) if comm is not None else \
            torch.empty(qkv.shape[0], num_heads, dtype=torch.float32, device=qkv.device)
        ext.attn_rowdot(out, dout, drow, num_heads)          # before the barrier that publishes this rank's rows
    if comm is None:
        dqkv = torch.empty_like(qkv)
        qkv_ptrs, dout_ptrs, dqkv_ptrs = [qkv.data_ptr()], [dout.data_ptr()], [dqkv.data_ptr()]
        if large:
            lse_ptrs, drow_ptrs = [lse.data_ptr()], [drow.data_ptr()]
    else:
        dqkv, qkv_ptrs, dout_ptrs, dqkv_ptrs = comm.attn_backward_buffers(qkv, dout, shifted)
        if large:
            lse_ptrs, drow_ptrs = comm.arena.peer_ptrs(lse), comm.arena.peer_ptrs(drow)
    launch_window_attn_bwd(ext, qkv_ptrs, dout_ptrs, dqkv_ptrs, bias_f32, dbias, geo, C, num_heads, sh, sw,
                           use_mask and shifted, scale, qkv.device, lse_ptrs, drow_ptrs)
    if comm is not None:
        dqkv = comm.attn_backward_done(dqkv, shifted)
    return dqkv


class _WindowAttnFn(torch.autograd.Function):
    """CUDA path. Without ``comm`` this rank owns every window and token. With a fused ``comm`` the q/k/v rows are
    staged in symmetric memory so that the kernels of the peer ranks can read them (and write outputs / gradients
    into this rank's rows) directly."""

    @staticmethod
    def forward(ctx, qkv, bias_table, geo, num_heads, shifted, use_mask, scale, comm):
        ext = _ext.load()
        C = qkv.shape[-1] // 3
        bias_f32 = fp32_values(bias_table).detach().float().contiguous() if bias_table is not None else None
        if comm is not None:
            staged = comm.alloc_qkv(qkv.shape[0], 3 * C)
            staged.copy_(qkv)
            qkv = staged
        out, qkv, lse = attention_forward(ext, qkv, geo, C, num_heads, shifted, use_mask, scale, bias_f32, comm)
        empty = torch.empty(0, device=qkv.device)
        ctx.save_for_backward(qkv, bias_f32 if bias_f32 is not None else empty, out, lse if lse is not None else empty)
        ctx.geo, ctx.num_heads, ctx.shifted, ctx.use_mask, ctx.scale, ctx.comm = geo, num_heads, shifted, use_mask, scale, comm
        ctx.has_bias = bias_table is not None
        return out

    @staticmethod
    def backward(ctx, dout):
        ext = _ext.load()
        qkv, bias_f32, out, lse = ctx.saved_tensors
        geo, comm = ctx.geo, ctx.comm
        C = qkv.shape[-1] // 3
        dout = dout.contiguous()
        dbias = torch.zeros_like(bias_f32) if ctx.has_bias else None
        if comm is not None:
            staged = comm.alloc_dout(dout.shape[0], C)
            staged.copy_(dout)
            dout = staged
        dqkv = attention_backward(ext, qkv, out, dout, lse if lse.numel() else None, geo, C, ctx.num_heads, ctx.shifted,
                                  ctx.use_mask, ctx.scale, bias_f32 if ctx.has_bias else None, dbias, comm)
        return dqkv, dbias, None, None, None, None, None, None


@nvtx_range("terra.window_attention")
def window_attention(qkv: torch.Tensor, geo: WindowGeometry, num_heads: int, shifted: bool,
                     bias_table: Optional[torch.Tensor], use_mask: bool, scale: float, comm=None) -> torch.Tensor:
    """``qkv``: ``[rows_local, 3C]`` -> ``[rows_local, C]``. ``comm`` supplies peer access for multi-rank layouts
    (``None``: this rank owns every window and token)."""
    fused = comm is None or getattr(comm, "fused", False)
    if qkv.is_cuda and fused:
        return _WindowAttnFn.apply(qkv, bias_table, geo, num_heads, shifted, use_mask, scale, comm)
    if comm is not None and comm.world > 1:
        return comm.window_attention_portable(qkv, geo, num_heads, shifted, bias_table, use_mask, scale)
    C = qkv.shape[-1] // 3
    out = window_attention_reference(qkv.reshape(geo.B, geo.nWh * geo.nWw, geo.N, 3 * C), geo, num_heads, shifted,
                                     bias_table, use_mask, scale)
    return out.reshape(-1, C)
