"""Python front end of the tcgen05 GEMM family.

``gemm`` computes ``epilogue(A_op @ B_op^T)`` where the stored orientation of each operand is a flag, so
that forward, input-gradient and weight-gradient products of a linear layer all run on the same kernel
without materialising a transpose:

    forward      y  = x  @ W^T          a=x  [M,K]         b=W  [N,K]
    input grad   dx = dy @ W            a=dy [M,N]         b=W  [N,K] read MN-major (b_mn=True)
    weight grad  dW = dy^T @ x          a=dy [M,N] (a_mn)  b=x  [M,K] (b_mn), split-K fp32 atomics

The reference reaches cuBLAS for these products through ``nn.Linear`` / ``torch.matmul`` (models/attention.py:766-793,
models/mlp.py:478-530, core/dist_matmul.py:8-459); here they are one hand-written kernel family (csrc/gemm_sm100.cu).
"""
from __future__ import annotations

import os
import sys
from typing import Optional, Sequence

import torch

from .. import _ext
from . import _flags as F
from ..utils.nvtx import nvtx_range

_status = {}
_TRACE = os.environ.get("TERRA_TRACE", "0") == "1"


def status_word(device) -> torch.Tensor:
    """Per-device 4 x uint32 record that kernels write when a bounded wait runs out."""
    key = torch.device(device).index or 0
    if key not in _status:
        _status[key] = torch.zeros(4, dtype=torch.int32, device=device)
        if _ext.DEBUG_BOUNDS and torch.device(device).type == "cuda":
            _ext.load().set_debug_status(_status[key])      # the attention kernels' location checks report here
    return _status[key]


def check_status(device) -> None:
    """Raise if any kernel since the last check reported a timed-out wait (synchronises)."""
    st = status_word(device).cpu().tolist()
    if st[0] != 0:
        status_word(device).zero_()
        raise RuntimeError(
            f"terra_b200 kernel reported error {st[0]} at site 0x{st[1] & 0xffffffff:x} (info {st[2]}, {st[3]})"
        )


@nvtx_range("terra.gemm")
def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    bias: Optional[torch.Tensor] = None,
    gelu: bool = False,
    save_pre: bool = False,
    residual: Optional[torch.Tensor] = None,
    dgelu_aux: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    out_f32: bool = False,
    accumulate: bool = False,
    split_k: int = 1,
    alpha: float = 1.0,
    bn: int = 0,
    sms: int = 0,
    a_peers: Optional[Sequence[int]] = None,
    rank: int = 0,
    out_peers: Optional[Sequence[int]] = None,
    a_flags: int = 0,
    a_epoch: int = 0,
    a_budget_ns: int = 0,
    a_interleave: bool = True,
    a_chunks: int = 1,
    colsum: Optional[torch.Tensor] = None,
):
    """Returns ``out`` (and the saved pre-activation when ``save_pre``).

    Tensor-parallel fusions over peer memory: with ``a_peers`` (device pointers of every GPU's ``[rows, K]`` shard in
    symmetric memory, ``a`` being this GPU's) the operand is the concatenation of the shards, fetched tile by tile over
    NVLink inside the GEMM (all-gather -> GEMM). With ``out_peers`` (pointers of every GPU's fp32 ``[M / n, N]``
    accumulation buffer, ``out`` being this GPU's) the result rows are reduced into their owner's buffer from the
    epilogue (GEMM -> reduce-scatter). With ``a_flags`` / ``a_epoch`` the kernel itself waits for each peer's
    "shard written" signal instead of a barrier in front of it. ``colsum`` (fp32, one entry per output row; the
    weight-gradient form ``a_mn and b_mn`` with ``accumulate``): the sums of ``a``'s columns over the contraction, i.e.
    the bias gradient, are accumulated into it by the same kernel. ``out_peers`` with a bf16 ``out`` (shape
    ``[n, M / n, N]``): plain stores into this GPU's slot of the owners' staging, which the owner sums."""
    ext = _ext.load()
    M = a.shape[1] if a_mn else a.shape[0]
    if a_peers is not None and len(a_peers) > 1:
        M *= len(a_peers)
    if out_peers is not None and len(out_peers) > 1 and (out is None or out.dtype == torch.float32):
        accumulate = True
    N = b.shape[1] if b_mn else b.shape[0]
    flags = 0
    if bias is not None:
        flags |= F.EPI_BIAS
        if bias.dtype == torch.float32:
            flags |= F.EPI_BIAS_F32
    if gelu:
        flags |= F.EPI_GELU
    if residual is not None:
        flags |= F.EPI_RESIDUAL
    if dgelu_aux is not None:
        flags |= F.EPI_MUL_DGELU
    if out_f32 or accumulate or split_k > 1:
        flags |= F.EPI_OUT_F32
    if accumulate or split_k > 1:
        flags |= F.EPI_ATOMIC
    if out is None:
        dt = torch.float32 if (flags & F.EPI_OUT_F32) else torch.bfloat16
        if flags & F.EPI_ATOMIC:
            out = torch.zeros(M, N, dtype=dt, device=a.device)
        else:
            out = torch.empty(M, N, dtype=dt, device=a.device)
    pre = None
    if save_pre:
        flags |= F.EPI_SAVE_PRE
        pre = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    if _TRACE:
        print(f"[terra trace] gemm a={tuple(a.shape)}/{a.dtype}/{a.stride()} a_mn={a_mn} b={tuple(b.shape)}/{b.dtype}/{b.stride()} "
              f"b_mn={b_mn} out={tuple(out.shape)}/{out.dtype}/{out.stride()}/{out.device} flags={flags} split_k={split_k} bn={bn} "
              f"bias={None if bias is None else (tuple(bias.shape), bias.dtype)} "
              f"res={None if residual is None else (tuple(residual.shape), residual.dtype, residual.stride())}",
              file=sys.stderr, flush=True)
    ext.gemm(a, a_mn, b, b_mn, out, flags, bias, residual, dgelu_aux, pre, float(alpha), int(split_k), int(bn),
             status_word(a.device), 0, 0, 0, int(sms), list(a_peers or []), int(rank), list(out_peers or []),
             int(a_flags), int(a_epoch), int(a_budget_ns), int(bool(a_interleave)), int(a_chunks), colsum)
    if save_pre:
        return out, pre
    return out
