"""Distributed ``Y = X W^T (+ b)`` over a model-parallel group in the four operand layouts of the reference's 2-D
distributed GEMM (core/dist_matmul.py:8-459; ``XWT_apply``: 449-459).

``input_split`` says how the activation ``X [tokens, in]`` is cut over the ``n`` ranks of the group, ``output_split`` how
the result ``Y [tokens, out]`` is:

  ``'(m,1)'``  by rows: every rank holds ``tokens / n`` consecutive rows and all columns;
  ``'(1,n)'``  by columns: every rank holds all rows and ``features / n`` consecutive columns.

The weight shard follows from the pair (``split_param``): a column shard ``W[:, in / n]`` where the activation is cut by
columns (the contraction is distributed, partial products are summed), a row shard ``W[out / n, :]`` where it is cut
by rows.

  input   output   weight shard      forward                                          traffic
  (1,n)   (m,1)    [out, in / n]     partial product, rows reduce-scattered           reduce-scatter of [tokens, out]
  (1,n)   (1,n)    [out, in / n]     partial product, columns reduce-scattered        reduce-scatter of [tokens, out]
  (m,1)   (m,1)    [out / n, in]     weight rows all-gathered, local product          all-gather of [out, in]
  (m,1)   (1,n)    [out / n, in]     activation rows all-gathered, local product      all-gather of [tokens, in]

Where the reference loops over the ranks with one broadcast or reduce per rank, each case here is one collective
written with the autograd-aware primitives of ``collectives.py``, so the input and weight gradients (the reference's
``dist_XW`` and ``dist_XTW``) are the adjoint collectives and need no second implementation: reduce-scatter <->
all-gather. Leading batch dimensions are folded into the rows. On B200 the two layouts the model uses, (m,1) ->
(1,n) and (1,n) -> (m,1), have fused kernels (all-gather -> GEMM and GEMM -> reduce-scatter over NVLink peer memory,
``ops/tp_fused.py``); this module is the portable form of all four and the oracle those kernels are tested against.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import collectives as C

LAYOUTS = ("(m,1)", "(1,n)")


def _check(input_split: str, output_split: str) -> None:
    if input_split not in LAYOUTS or output_split not in LAYOUTS:
        raise ValueError(f"dist_matmul: splits must be '(m,1)' or '(1,n)', got {input_split!r} -> {output_split!r}")


def _matmul_t(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x @ w^T`` for 2-D operands through ``torch.matmul`` (differentiable on every device; this module is the portable
    form, the fused sm_100a kernels live in ``ops/tp_fused.py``)."""
    return torch.matmul(x, w.transpose(-1, -2))


def _columns_to_rows(y: torch.Tensor, n: int) -> torch.Tensor:
    """[rows, n * c] -> [n * rows, c]: column block j becomes row block j (so that a row collective moves columns)."""
    rows, cols = y.shape
    return y.reshape(rows, n, cols // n).transpose(0, 1).reshape(n * rows, cols // n)


def _rows_to_columns(y: torch.Tensor, n: int) -> torch.Tensor:
    rows, c = y.shape[0] // n, y.shape[1]
    return y.reshape(n, rows, c).transpose(0, 1).reshape(rows, n * c)


def dist_xwt(x: torch.Tensor, w: torch.Tensor, group, input_split: str, output_split: str,
             bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``Y = X W^T (+ bias)`` with ``x`` and ``w`` this rank's shards (see the module docstring); returns this rank's
    shard of ``Y`` in ``output_split``. ``bias`` is this rank's part of the bias for the columns it returns (the whole
    bias for ``(m,1)`` outputs, ``out / n`` entries for ``(1,n)``). Differentiable in ``x``, ``w`` and ``bias``."""
    _check(input_split, output_split)
    n = C.group_size(group)
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if input_split == "(1,n)":
        part = _matmul_t(x2, w)                                   # [tokens, out], partial over the contraction shards
        if output_split == "(m,1)":
            if part.shape[0] % n:
                raise ValueError(f"dist_matmul: {part.shape[0]} rows do not split over {n} ranks")
            y = C.reduce_scatter_rows(part, group)
            lead = None
        else:
            if part.shape[1] % n:
                raise ValueError(f"dist_matmul: {part.shape[1]} output features do not split over {n} ranks")
            y = C.reduce_scatter_rows(_columns_to_rows(part, n), group) if n > 1 else part
    else:
        if output_split == "(m,1)":
            y = _matmul_t(x2, C.all_gather_rows(w, group))         # every rank needs the whole weight
        else:
            y = _matmul_t(C.all_gather_rows(x2, group), w)         # every rank needs every row
            lead = None
    if bias is not None:
        y = y + bias.to(y.dtype)
    return y if lead is None else y.reshape(*lead, y.shape[-1])


def xwt_apply(x, weight, bias, group, input_split: str, output_split: str, use_bias: bool = True):
    """Call-compatible counterpart of the reference's ``XWT_apply`` with the process group in place of the manager."""
    return dist_xwt(x, weight, group, input_split, output_split, bias if use_bias else None)


def full_reference(x_full: torch.Tensor, w_full: torch.Tensor, bias_full: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The undistributed product, for tests."""
    y = torch.matmul(x_full, w_full.transpose(-1, -2))
    return y if bias_full is None else y + bias_full


def shard(t: torch.Tensor, split: str, rank: int, n: int) -> torch.Tensor:
    """This rank's part of a full ``[rows, cols]`` matrix in layout ``split``."""
    if split == "(m,1)":
        per = t.shape[0] // n
        return t[rank * per:(rank + 1) * per]
    per = t.shape[1] // n
    return t[:, rank * per:(rank + 1) * per]
